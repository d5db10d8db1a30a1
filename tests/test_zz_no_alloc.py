"""tri_decode_static: the decode step for callers that cannot allocate device memory.

Such a caller (a serving runtime that handed all of HBM to its KV pool at start-up, or a language binding
that can only forward buffers it was given) has nowhere to put the split-KV partials that tri_decode
expects from its caller.  tri_decode_static keeps them in a fixed array inside the library.  This file
checks, through the C ABI, that two calls in a row give bit for bit what tri_decode gives on the same inputs
(same kernels, same plan), that a plan too large for the fixed array is refused, and that a plan whose slot
numbers point outside the array is caught by the kernels' own bounds check (error word 4, nothing stored there)
rather than written past the array.  It is collected last on purpose: a run that stops at the first failure
has already run every other test.
"""
import numpy as np
import pytest
import torch

from triattention_b200.kernels.decode import DecodeCache
from triattention_b200.kernels.prefill import Prefill
from triattention_b200.maps import INF, from_bands
from util import assert_fp_close, bf16_cuda, make_inputs

pytestmark = pytest.mark.gpu
SCALE = 1.0 / np.sqrt(128.0)


def build(module, hq, hk, t, bands, batch, seed, bf16=()):
    fn = from_bands({"0": np.asarray(bands).tolist()}, None, {"0": list(bf16)} if bf16 else None)
    cache = DecodeCache(module, max_tail=8)
    pre = Prefill(module, fn, cache)
    q, k, v = make_inputs(hq, hk, t, seed=seed, batch=batch)
    kc, vc = bf16_cuda(k), bf16_cuda(v)
    table, ops = pre.write(0, bf16_cuda(q), kc, vc)
    cache.store(0, t, ops, table.host, kc, vc, table.bf16_kv)
    return cache


def static_step(module, cache, q, k, v, segments=None, unit_slots=None):
    e, d = cache.layers[0], cache.layers[0]["dev"]
    out = torch.zeros_like(q)
    module.decode_static(q, e["pool"], d["unit_base"], d["unit_tab"], d["unit_flags"], d["tmeta"],
                         d["segments"] if segments is None else segments, d["cta_segments"],
                         d["unit_slots"] if unit_slots is None else unit_slots, e["kstat"], e["vstat"], e["tail_k"],
                         e["tail_v"], k, v, cache.step, out, e["prompt"], SCALE)
    return out


def test_two_calls_match_the_allocating_entry_point(module):
    hq, hk, t, batch = 6, 3, 1500, 2
    bands = [[INF, INF]] * 2 + [[4, 12]] * 2 + [[INF, INF]] * 2
    cache = build(module, hq, hk, t, bands, batch, seed=7, bf16=(2,))
    qd, kd, vd = make_inputs(hq, hk, 2, seed=8, batch=batch)
    for s in range(2):   # two calls in a row share the library's array; the second must not see the first
        q, k, v = (bf16_cuda(x[:, :, s:s + 1]) for x in (qd, kd, vd))
        want = cache(0, q, k, v, SCALE).float().cpu().numpy()
        got = static_step(module, cache, q, k, v).float().cpu().numpy()
        module.check_device_error()
        assert np.isfinite(got).all()
        assert_fp_close(got, want, f"static decode, call {s}")
        assert (got == want).all(), f"static decode, call {s}: not bit-equal to tri_decode"
        cache.advance()


def test_plans_beyond_the_fixed_array_are_refused(module):
    hq, hk, t, batch = 2, 2, 64, 600          # 1200 one-tile units -> 1200 partial slots > 1024
    cache = build(module, hq, hk, t, [[INF, INF]] * 2, batch, seed=9)
    assert cache.layers[0]["plan"]["slots"] > 1024
    q, k, v = (bf16_cuda(x) for x in make_inputs(hq, hk, 1, seed=10, batch=batch))
    with pytest.raises(RuntimeError, match="1024 partial slots"):
        static_step(module, cache, q, k, v)
    cache(0, q, k, v, SCALE)                 # the allocating entry point still takes it
    module.check_device_error()


def test_slot_numbers_outside_the_array_are_caught_on_the_device(module):
    """A caller-built plan whose slot column is not 0 .. num_slots-1: the host check sees only the number of rows, so
    the kernels compare every slot with the array's capacity, skip the access and report error 4."""
    hq, hk, t, batch = 4, 2, 300, 2
    cache = build(module, hq, hk, t, [[INF, INF]] * 4, batch, seed=11)
    q, k, v = (bf16_cuda(x) for x in make_inputs(hq, hk, 1, seed=12, batch=batch))
    d = cache.layers[0]["dev"]
    want = static_step(module, cache, q, k, v)
    module.check_device_error()
    for shift_segments, shift_units in ((True, True), (False, True)):
        segments, unit_slots = d["segments"].clone(), d["unit_slots"].clone()
        if shift_segments:
            segments[:, 3] += 1 << 20           # far beyond the 1024 slots of the array
        if shift_units:
            unit_slots[:, 0] += 1 << 20
        static_step(module, cache, q, k, v, segments, unit_slots)
        with pytest.raises(RuntimeError, match="device error 4"):
            module.check_device_error()
    again = static_step(module, cache, q, k, v)     # the library and the array are intact afterwards
    module.check_device_error()
    assert torch.equal(again, want)
