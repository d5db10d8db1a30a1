"""Split-KV decode + merge against the CPU oracle and the reference extension."""
import numpy as np
import pytest
import torch

import triattention_oracle as orc
from ref_harness import RefRunner
from triattention_b200.kernels.decode import DecodeCache
from triattention_b200.kernels.prefill import Prefill
from triattention_b200.maps import INF, from_bands
from util import assert_fp_close, bf16_cuda, make_inputs

pytestmark = pytest.mark.gpu
SCALE = 1.0 / np.sqrt(128.0)


def bands_fn_of(bands, bf16=()):
    fn = from_bands({"0": np.asarray(bands).tolist()}, None, {"0": list(bf16)} if bf16 else None)
    return fn


def product_decode(module, q, k, v, bands, qd, kd, vd, steps, max_tail=8, bf16=(), fused=False, ctas=None):
    """Write the cache with the product path, then run `steps` decode steps.  Arrays are [B,H,*,128]."""
    cache = DecodeCache(module, max_tail=max_tail, fused_merge=fused, ctas=ctas)
    pre = Prefill(module, bands_fn_of(bands, bf16), cache)
    kc, vc = bf16_cuda(k), bf16_cuda(v)
    table, ops = pre.write(0, bf16_cuda(q), kc, vc)
    cache.store(0, q.shape[2], ops, table.host, kc, vc, table.bf16_kv)
    outs = []
    for s in range(steps):
        out = cache(0, bf16_cuda(qd[:, :, s:s + 1]), bf16_cuda(kd[:, :, s:s + 1]), bf16_cuda(vd[:, :, s:s + 1]), SCALE)
        cache.advance()
        outs.append(out.float().cpu().numpy()[:, :, 0])
    module.check_device_error()
    return np.stack(outs, 1), cache      # [B, steps, Hq, 128]


def oracle_ops(q, k, v):
    kstat = orc.channel_stats(k)
    k8, ka, k4, ka4 = orc.quantize_k(k, kstat[:, 0])
    vstat = orc.channel_stats(v)
    v16, v8, v4 = orc.pack_v(v, vstat)
    return dict(kstat=kstat, k8=k8, ka=ka, k4=k4, ka4=ka4, vstat=vstat, v16=v16, v8=v8, v4=v4)


def oracle_steps(k, v, bands, qd, kd, vd, steps, max_tail=8, per=None):
    """One sequence: [H,T,128] arrays -> [steps, Hq, 128] float32."""
    ops = oracle_ops(None, k, v)
    hk = k.shape[0]
    tk, tv = np.zeros((hk, max_tail, 128), np.float32), np.zeros((hk, max_tail, 128), np.float32)
    outs = []
    for s in range(steps):
        outs.append(orc.decode_step(qd[:, s], ops, bands, k.shape[1], SCALE, tk, tv, kd[:, s], vd[:, s], s, max_tail, per))
    return np.stack(outs)


CASES = [
    # hq, hk, t, bands
    (4, 2, 200, [[INF, INF], [INF, INF], [2, 3], [2, 3]]),
    (8, 2, 512, [[INF, INF]] * 4 + [[1, INF]] * 4),
    (6, 2, 1500, [[INF, INF]] * 3 + [[4, 12]] * 2 + [[1, 2]]),     # INT4 V tiles, dropped tiles, mixed row masks
    (3, 1, 65, [[INF, INF]] * 3),
    (8, 1, 130, [[1, INF]] * 8),
]


@pytest.mark.parametrize("fused", [True, False], ids=["one-launch", "two-launches"])
@pytest.mark.parametrize("hq,hk,t,bands", CASES)
def test_decode_vs_oracle(module, hq, hk, t, bands, fused):
    bands = np.asarray(bands, np.int64)
    q, k, v = make_inputs(hq, hk, t, seed=31, batch=2)
    qd, kd, vd = make_inputs(hq, hk, 3, seed=77, batch=2)
    got, cache = product_decode(module, q, k, v, bands, qd, kd, vd, steps=3, fused=fused)
    assert (cache.layers[0]["unit_done"] is not None) == fused
    if fused:   # the completion counters are back at zero after every step
        assert int(cache.layers[0]["unit_done"].abs().sum()) == 0
    for b in range(2):
        want = oracle_steps(k[b], v[b], bands, qd[b], kd[b], vd[b], 3)
        assert_fp_close(got[b], orc.to_bf16(want), f"decode b={b}")


@pytest.mark.parametrize("hq,hk,t,bands", CASES)
def test_decode_vs_reference(module, ref_ext, hq, hk, t, bands):
    bands = np.asarray(bands, np.int64)
    q, k, v = make_inputs(hq, hk, t, seed=41, batch=1)
    qd, kd, vd = make_inputs(hq, hk, 3, seed=88, batch=1)
    got, _ = product_decode(module, q, k, v, bands, qd, kd, vd, steps=3)
    run = RefRunner(ref_ext)
    o = run.prefill(bf16_cuda(q[0])[None], bf16_cuda(k[0])[None], bf16_cuda(v[0])[None], bands, SCALE)
    st = run.decode_setup(o, bands, max_tail=8, per=3)
    for s in range(3):
        ref = run.decode(st, bf16_cuda(qd[:, :, s:s + 1]), bf16_cuda(kd[:, :, s:s + 1]), bf16_cuda(vd[:, :, s:s + 1]), SCALE)
        st["step"].add_(1)
        assert_fp_close(got[0, s], ref.float().cpu().numpy()[0, :, 0], f"decode step {s}")


def test_decode_bf16_heads(module):
    """Un-quantised extension heads against exact attention over prompt + tail."""
    hq, hk, t = 6, 3, 300
    bands = np.asarray([[INF, INF]] * 6, np.int64)
    q, k, v = make_inputs(hq, hk, t, seed=51, batch=2)
    qd, kd, vd = make_inputs(hq, hk, 2, seed=99, batch=2)
    got, _ = product_decode(module, q, k, v, bands, qd, kd, vd, steps=2, bf16=(1,))
    for b in range(2):
        for s in range(2):
            for h in (2, 3):
                kk = np.concatenate([k[b, 1], kd[b, 1, :s + 1]])
                vv = np.concatenate([v[b, 1], vd[b, 1, :s + 1]])
                want = orc.exact_decode(qd[b, h, s], kk, vv, SCALE)
                assert_fp_close(got[b, s, h], orc.to_bf16(want), f"bf16 head {h} step {s}")
        # quantised heads in the same launch still match the oracle
        want = oracle_steps(k[b], v[b], bands, qd[b], kd[b], vd[b], 2)
        assert_fp_close(got[b][:, [0, 1, 4, 5]], orc.to_bf16(want[:, [0, 1, 4, 5]]), "mixed launch")


def test_decode_split_invariance(module):
    """The work-list cut must not change the result beyond float summation order."""
    from triattention_b200.kernels import decode as dm
    hq, hk, t = 4, 2, 2000
    bands = np.asarray([[INF, INF]] * 4, np.int64)
    q, k, v = make_inputs(hq, hk, t, seed=61)
    qd, kd, vd = make_inputs(hq, hk, 1, seed=62)
    results = []
    for ctas in (1, 16, 444):
        cache = DecodeCache(module, max_tail=4, ctas=ctas)
        pre = Prefill(module, bands_fn_of(bands), cache)
        kc, vc = bf16_cuda(k), bf16_cuda(v)
        table, ops = pre.write(0, bf16_cuda(q), kc, vc)
        cache.store(0, t, ops, table.host, kc, vc)
        results.append(cache(0, bf16_cuda(qd), bf16_cuda(kd), bf16_cuda(vd), SCALE).float().cpu().numpy())
    module.check_device_error()
    assert_fp_close(results[1], results[0], "16 CTAs vs 1")
    assert_fp_close(results[2], results[0], "444 CTAs vs 1")


@pytest.mark.parametrize("ctas", [3, 148, 444])
def test_fused_merge_matches_two_launches(module, ctas):
    """The merge done by the last CTA of a unit against the separate merge launch, with units cut into many
    segments and CTAs that own several units, over enough steps to reuse the completion counters."""
    hq, hk, t = 8, 2, 3000
    bands = np.asarray([[INF, INF]] * 4 + [[2, 6]] * 4, np.int64)
    q, k, v = make_inputs(hq, hk, t, seed=63, batch=3)
    qd, kd, vd = make_inputs(hq, hk, 6, seed=64, batch=3)
    one, _ = product_decode(module, q, k, v, bands, qd, kd, vd, steps=6, max_tail=4, fused=True, ctas=ctas)
    two, _ = product_decode(module, q, k, v, bands, qd, kd, vd, steps=6, max_tail=4, fused=False, ctas=ctas)
    assert_fp_close(one, two, f"one launch vs two, {ctas} CTAs")


@pytest.mark.parametrize("fused,hq,hk", [(True, 8, 2), (False, 8, 2), (False, 6, 2), (False, 7, 1), (False, 16, 2)],
                         ids=["one-launch", "two-launches", "group-of-3", "group-of-7", "group-of-8"])
def test_long_tail_merge_kernel_gives_the_same_bits(module, monkeypatch, fused, hq, hk):
    """The merge kernel has a second instantiation for long BF16 tails (row loops unrolled), which the host picks from
    its count of generated tokens (tri_decode_tail_hint).  70 steps with the hint as DecodeCache gives it (plain kernel up
    to 8 rows, unrolled after), with the plain kernel throughout and with the unrolled one throughout: the same bits,
    and the oracle's values.  The unrolled kernel reduces the scores of four Q heads of a group at a time, so groups
    of 3, 4, 7 and 8 heads are run."""
    t, steps = 300, 70
    bands = np.asarray([[INF, INF]] * (hq // 2) + [[2, 6]] * (hq - hq // 2), np.int64)
    q, k, v = make_inputs(hq, hk, t, seed=73, batch=2)
    qd, kd, vd = make_inputs(hq, hk, steps, seed=74, batch=2)
    hints = []
    hint = module.decode_tail_hint
    monkeypatch.setattr(module, "decode_tail_hint", lambda rows: (hints.append(rows), hint(rows))[1])
    as_counted, _ = product_decode(module, q, k, v, bands, qd, kd, vd, steps=steps, max_tail=128, fused=fused)
    assert hints == list(range(1, steps + 1))
    for rows in (1, 1000):
        monkeypatch.setattr(DecodeCache, "tail_rows", lambda self: rows)
        forced, _ = product_decode(module, q, k, v, bands, qd, kd, vd, steps=steps, max_tail=128, fused=fused)
        assert np.array_equal(as_counted, forced), rows
    monkeypatch.undo()
    module.decode_tail_hint(-1)
    want = oracle_steps(k[0], v[0], bands, qd[0], kd[0], vd[0], steps, max_tail=128)
    assert_fp_close(as_counted[0], orc.to_bf16(want), "70-row tail")
    # Past the 256 rows that the unrolled kernel copies into shared memory (the rest it reads where they lie), and into
    # the saturated tail: 290 steps on a tail of at most 280 rows.
    qd, kd, vd = make_inputs(hq, hk, 290, seed=75, batch=2)
    runs = []
    for rows in (1, 1000):
        monkeypatch.setattr(DecodeCache, "tail_rows", lambda self: rows)
        runs.append(product_decode(module, q, k, v, bands, qd, kd, vd, steps=290, max_tail=280, fused=fused)[0])
    monkeypatch.undo()
    module.decode_tail_hint(-1)
    assert np.array_equal(runs[0], runs[1])


def test_tail_saturates(module):
    """Steps beyond max_tail-1 keep overwriting the last tail slot (common_device.cuh:384)."""
    hq, hk, t = 2, 1, 64
    bands = np.asarray([[INF, INF]] * 2, np.int64)
    q, k, v = make_inputs(hq, hk, t, seed=71)
    qd, kd, vd = make_inputs(hq, hk, 4, seed=72)
    got, _ = product_decode(module, q, k, v, bands, qd, kd, vd, steps=4, max_tail=2)
    want = oracle_steps(k[0], v[0], bands, qd[0], kd[0], vd[0], 4, max_tail=2)
    assert_fp_close(got[0], orc.to_bf16(want), "saturated tail")


def test_host_stepper_matches_device_calls(module):
    """Pinned host buffers through the rotating device buffers give the same bits as device-resident calls,
    for more steps than there are buffer sets and with a different input every step."""
    from triattention_b200.kernels.decode import HostStepper
    hq, hk, t, steps = 4, 2, 700, 5
    bands = np.asarray([[INF, INF], [INF, INF], [3, 5], [3, 5]], np.int64)
    q, k, v = make_inputs(hq, hk, t, seed=81, batch=2)
    qd, kd, vd = make_inputs(hq, hk, steps, seed=82, batch=2)
    want, _ = product_decode(module, q, k, v, bands, qd, kd, vd, steps=steps)
    cache = DecodeCache(module, max_tail=8)
    pre = Prefill(module, bands_fn_of(bands), cache)
    kc, vc = bf16_cuda(k), bf16_cuda(v)
    table, ops = pre.write(0, bf16_cuda(q), kc, vc)
    cache.store(0, t, ops, table.host, kc, vc)
    pin = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(torch.bfloat16).pin_memory()
    stepper = HostStepper(cache, 0, (2, hq, 1, 128), (2, hk, 1, 128), "cuda")
    outs = [torch.empty((2, hq, 1, 128), dtype=torch.bfloat16).pin_memory() for _ in range(steps)]
    for s in range(steps):
        stepper.submit(pin(qd[:, :, s:s + 1]), pin(kd[:, :, s:s + 1]), pin(vd[:, :, s:s + 1]), outs[s], SCALE)
        cache.advance()
    stepper.wait()
    module.check_device_error()
    got = np.stack([o.float().numpy()[:, :, 0] for o in outs], 1)
    np.testing.assert_array_equal(got, want)
    with pytest.raises(RuntimeError):
        stepper.submit(torch.empty(1), outs[0], outs[0], outs[0], SCALE)


def test_fold_tail_lifts_the_generation_cap(module):
    """DecodeCache(fold_tail=N): every 64 generated tokens become one more cached tile (quantised with the prompt's
    statistics), so generation runs past max_tail.  Quantised heads against the oracle's restatement of exactly
    that, BF16 units against exact attention over all keys; 131 steps = two folds, ragged prompt end."""
    hq, hk, t, steps = 6, 3, 200, 131
    bands = np.asarray([[INF, INF]] * 2 + [[1, INF]] * 2 + [[INF, INF]] * 2, np.int64)
    q, k, v = make_inputs(hq, hk, t, seed=71, batch=2)
    qd, kd, vd = make_inputs(hq, hk, steps, seed=72, batch=2)
    cache = DecodeCache(module, max_tail=64, fold_tail=192)
    pre = Prefill(module, bands_fn_of(bands, (2,)), cache)
    kc, vc = bf16_cuda(k), bf16_cuda(v)
    table, ops = pre.write(0, bf16_cuda(q), kc, vc)
    cache.store(0, t, ops, table.host, kc, vc, table.bf16_kv)
    got = []
    for s in range(steps):
        got.append(cache(0, bf16_cuda(qd[:, :, s:s + 1]), bf16_cuda(kd[:, :, s:s + 1]), bf16_cuda(vd[:, :, s:s + 1]),
                         SCALE).float().cpu().numpy()[:, :, 0])
        cache.advance()
    module.check_device_error()
    assert cache.layers[0]["extra"] == 2 and int(cache.step) == steps % 64
    got = np.stack(got, 1)
    for b in range(2):
        o = oracle_ops(None, k[b], v[b])
        tk, tv = np.zeros((hk, 64, 128), np.float32), np.zeros((hk, 64, 128), np.float32)
        appended = []
        for s in range(steps):
            if s and s % 64 == 0:
                appended.append(orc.fold_tail(o, tk.copy(), tv.copy()))
            want = orc.decode_step(qd[b][:, s], o, bands, t, SCALE, tk, tv, kd[b][:, s], vd[b][:, s], s % 64, 64,
                                   appended=appended)
            assert_fp_close(got[b, s, :4], orc.to_bf16(want[:4]), f"b={b} step {s}")
            for h in (4, 5):
                kk, vv = np.concatenate([k[b, 2], kd[b, 2, :s + 1]]), np.concatenate([v[b, 2], vd[b, 2, :s + 1]])
                assert_fp_close(got[b, s, h], orc.to_bf16(orc.exact_decode(qd[b, h, s], kk, vv, SCALE)), f"bf16 head {h} step {s}")
    # against the un-folded cache (all generated tokens in the BF16 tail) only the 128 folded keys differ: INT8 codes
    plain, _ = product_decode(module, q, k, v, bands, qd, kd, vd, steps, max_tail=256, bf16=(2,))
    # (the softmax of these inputs is peaked, so INT8 logits move single elements by a few tenths; the check is that
    # the two stay the same attention overall)
    a, b = plain[:, 64:].astype(np.float64).ravel(), got[:, 64:].astype(np.float64).ravel()
    assert np.array_equal(plain[:, :64], got[:, :64]) and a @ b / np.sqrt((a @ a) * (b @ b)) > 0.99
    # the reserved room is a hard limit
    small = DecodeCache(module, max_tail=64, fold_tail=64)
    pre = Prefill(module, bands_fn_of(bands, (2,)), small)
    table, ops = pre.write(0, bf16_cuda(q), kc, vc)
    small.store(0, t, ops, table.host, kc, vc, table.bf16_kv)
    small.generated = 128
    with pytest.raises(RuntimeError):
        small.fold(0), small.fold(0)


def test_store_in_parts_equals_store_at_once(module):
    """A cache filled one group of sequences at a time (long prompts) holds the same bytes and statistics."""
    hq, hk, t, batch = 6, 3, 330, 4
    bands = np.asarray([[INF, INF]] * 2 + [[1, INF]] * 2 + [[INF, INF]] * 2, np.int64)
    q, k, v = make_inputs(hq, hk, t, seed=81, batch=batch)
    qd, kd, vd = make_inputs(hq, hk, 1, seed=82, batch=batch)
    kc, vc, qc = bf16_cuda(k), bf16_cuda(v), bf16_cuda(q)
    whole = DecodeCache(module, max_tail=4)
    pre = Prefill(module, bands_fn_of(bands, (2,)), whole)
    table, ops = pre.write(0, qc, kc, vc)
    whole.store(0, t, ops, table.host, kc, vc, table.bf16_kv)
    parts = DecodeCache(module, max_tail=4)
    pre2 = Prefill(module, bands_fn_of(bands, (2,)), parts)
    for first, n in ((0, 1), (1, 2), (3, 1)):
        sl = slice(first, first + n)
        table, ops = pre2.write(0, qc[sl], kc[sl], vc[sl])
        parts.store(0, t, ops, table.host, kc[sl], vc[sl], table.bf16_kv, first_sequence=first, sequences=batch)
    a, b = whole.layers[0], parts.layers[0]
    assert torch.equal(a["kstat"], b["kstat"]) and torch.equal(a["vstat"], b["vstat"])
    plan = a["plan"]
    for unit, base in enumerate(plan["unit_base"]):            # every unit's stream, without the alignment padding behind it
        used = int(plan["append_off"][unit % hk])
        assert torch.equal(a["pool"][int(base):int(base) + used], b["pool"][int(base):int(base) + used]), unit
    args = (0, bf16_cuda(qd), bf16_cuda(kd), bf16_cuda(vd), SCALE)
    assert torch.equal(whole(*args), parts(*args))
    module.check_device_error()
    with pytest.raises(RuntimeError):
        DecodeCache(module, max_tail=4).store(0, t, ops, table.host, kc[3:], vc[3:], table.bf16_kv, first_sequence=3, sequences=batch)


@pytest.fixture(params=["merge-for-short-tails", "merge-for-long-tails"])
def merge_kernel(request, monkeypatch):
    """Runs a test once with the merge kernel that DecodeCache's row count picks (a few steps: the one for short tails)
    and once with the one for long tails (no hint given), which takes its tail rows through shared memory."""
    if request.param == "merge-for-long-tails":
        monkeypatch.setattr(DecodeCache, "tail_rows", lambda self: -1)
    return request.param


@pytest.mark.parametrize("exchange", ["nccl", "peer"])
@pytest.mark.parametrize("world,ctas", [(2, None), (3, 5), (8, None)])
def test_sequence_split_emulated_on_one_gpu(module, world, ctas, exchange, merge_kernel):
    """The sequence-split path without a process group: `world` caches each hold one part of every unit's tile range
    (what the ranks of a split group hold) and each runs its split pass with the in-kernel fold (tri_decode_partials).
    "nccl": the folded triples are stacked [rank][m | l | o] as an all-gather would leave them, and tri_decode_merge
    reads that buffer in place by stride.  "peer": every part's fold writes its triples, then a flag, straight into the
    exchange buffers of all parts (here all on this GPU), and the merge takes them from there; all producers are
    launched before any consumer, on one stream, so no kernel ever waits for another.
    Against the un-split decode over three steps, with a BF16 unit, an INT4 band and a prompt short enough that some
    parts hold no tile of some units."""
    hq, hk, t, batch = 6, 3, 900, 2
    bands = np.asarray([[INF, INF]] * 2 + [[2, 5]] * 2 + [[INF, INF]] * 2, np.int64)
    q, k, v = make_inputs(hq, hk, t, seed=71, batch=batch)
    qd, kd, vd = make_inputs(hq, hk, 3, seed=72, batch=batch)
    whole, _ = product_decode(module, q, k, v, bands, qd, kd, vd, steps=3, bf16=(2,))
    kc, vc = bf16_cuda(k), bf16_cuda(v)
    caches = []
    for rank in range(world):
        cache = DecodeCache(module, max_tail=8, split=(rank, world), ctas=ctas, exchange=exchange)
        pre = Prefill(module, bands_fn_of(bands, (2,)), cache)
        table, ops = pre.write(0, bf16_cuda(q), kc, vc)
        cache.store(0, t, ops, table.host, kc, vc, table.bf16_kv)
        caches.append(cache)
    if exchange == "peer":
        for cache in caches:
            cache.attach_peers(0, [c.layers[0]["xbuf"] for c in caches])
    g = hq // hk
    outs = []
    for s in range(3):
        qs, ks, vs = (bf16_cuda(x[:, :, s:s + 1]) for x in (qd, kd, vd))
        folded = []
        for cache in caches:            # every producer first
            e = cache.layers[0]
            mine = cache.partials(0, qs, ks, SCALE).clone()
            if exchange == "nccl":
                # the fused fold equals the stand-alone fold kernel bit for bit (same arithmetic, same order); rows of Q heads
                # the group does not have are written by neither
                fm, fl, fo = torch.empty_like(e["fm"]), torch.empty_like(e["fl"]), torch.empty_like(e["fo"])
                module.decode_fold(e["pm"], e["pl"], e["po"], e["dev"]["unit_slots"], fm, fl, fo, g)
                assert torch.equal(fm[:, :g], e["fm"][:, :g]) and torch.equal(fl[:, :g], e["fl"][:, :g])
                assert torch.equal(fo[:, :g], e["fo"][:, :g])
            folded.append(mine)
        outs_rank = []
        for cache in caches:        # every rank merges the same triples with its own (replicated) tail
            if exchange == "nccl":
                cache.layers[0]["gathered"].copy_(torch.stack(folded))
            outs_rank.append(cache.merge_gathered(0, qs, ks, vs, SCALE).float().cpu().numpy()[:, :, 0])
            cache.advance()
        assert all((o == outs_rank[0]).all() for o in outs_rank)
        outs.append(outs_rank[0])
    module.check_device_error()
    if exchange == "peer":          # every unit's counters moved once per step, on both sides
        for cache in caches:
            e = cache.layers[0]
            assert (e["seen"] == 3).all() and (e["epoch"][e["present"][cache.split[0]].bool()] == 3).all()
    assert_fp_close(np.stack(outs, 1), whole, f"sequence split over {world} parts vs whole units")


def test_exchange_wait_runs_out_without_hanging(module, merge_kernel):
    """The consumer's wait is bounded: a merge whose peers never deliver (nothing sets the flags) gives up after its time
    limit, reports device error 1 and leaves the context usable."""
    hq, hk, t, batch = 4, 2, 300, 1
    bands = np.asarray([[INF, INF]] * 4, np.int64)
    q, k, v = make_inputs(hq, hk, t, seed=73, batch=batch)
    qd, kd, vd = (bf16_cuda(x) for x in make_inputs(hq, hk, 1, seed=74, batch=batch))
    cache = DecodeCache(module, max_tail=8, split=(0, 2), exchange="peer")
    pre = Prefill(module, bands_fn_of(bands), cache)
    kc, vc = bf16_cuda(k), bf16_cuda(v)
    table, ops = pre.write(0, bf16_cuda(q), kc, vc)
    cache.store(0, t, ops, table.host, kc, vc, table.bf16_kv)
    other = torch.zeros_like(cache.layers[0]["xbuf"])      # stands for the absent rank's buffer: written, never read
    cache.attach_peers(0, [cache.layers[0]["xbuf"], other])
    cache.partials(0, qd, kd, SCALE)                       # this rank delivers; rank 1 never does
    cache.merge_gathered(0, qd, kd, vd, SCALE)
    with pytest.raises(RuntimeError, match="device error 1"):
        module.check_device_error()
    assert int(cache.layers[0]["seen"].max()) == 0          # nothing was merged
    whole, _ = product_decode(module, q, k, v, bands, *make_inputs(hq, hk, 1, seed=74, batch=batch), steps=1)
    assert np.isfinite(whole).all()                         # and the GPU still computes


@pytest.mark.parametrize("layout", ["two-parts", "eight-parts"])
def test_output_gather_by_peer_stores_emulated_on_one_gpu(module, layout, merge_kernel):
    """Units sharded over two (or eight) "ranks" held by this process on one GPU: each part's merge kernel stores its output rows into
    the full output tensor of both parts (their gather buffers, here ordinary device memory), the last CTA raises the
    part's flag in both, and the wait kernel of each part then finds both flags set (all producers are launched before any
    consumer, so nothing ever waits for a later launch).  The full tensor equals the un-sharded decode, bit for bit per
    row (a shard is the same units with its own CTA partition, so only the float summation order may differ: tolerance),
    over three steps so that both parity blocks are used."""
    from triattention_b200 import sharding
    hq, hk, t, batch, g = 8, 4, 700, 2, 2
    bands = np.asarray([[INF, INF]] * 4 + [[2, 5]] * 2 + [[1, INF]] * 2, np.int64)
    q, k, v = make_inputs(hq, hk, t, seed=81, batch=batch)
    qd, kd, vd = make_inputs(hq, hk, 3, seed=82, batch=batch)
    whole, _ = product_decode(module, q, k, v, bands, qd, kd, vd, steps=3)
    if layout == "two-parts":
        shards = [sharding.Shard(0, slice(0, 2), (0, 3)), sharding.Shard(1, slice(0, 2), (1, 2))]     # head groups, not in order
    else:       # one (sequence, KV head) unit per part, as an 8-GPU placement of few heavy units gives
        shards = [sharding.Shard(r, slice(r // 4, r // 4 + 1), ((r * 3) % 4,)) for r in range(8)]
    nbytes = sharding.PeerOutputGatherer.buffer_bytes(batch, hq, len(shards))
    fn = bands_fn_of(bands)
    buffers = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in shards]
    parts = []
    for s in shards:
        heads, qh = list(s.kv_heads), list(s.q_heads(g))
        cache = DecodeCache(module, max_tail=8)
        pre = Prefill(module, sharding.slice_map(fn, s, g, hq), cache)
        take = lambda x, hs, s=s: bf16_cuda(np.ascontiguousarray(x[s.batch][:, hs]))
        table, ops = pre.write(0, take(q, qh), take(k, heads), take(v, heads))
        cache.store(0, t, ops, table.host, take(k, heads), take(v, heads), table.bf16_kv)
        gather = sharding.PeerOutputGatherer(module, shards, g, batch, hq, "cuda", rank=s.rank, buffers=buffers)
        parts.append((cache, gather, heads, qh, s.batch))
    outs = []
    for step in range(3):
        for cache, gather, heads, qh, seqs in parts:          # every producer first: split pass + merge with peer stores
            e, d = cache.layers[0], cache.layers[0]["dev"]
            qs, ks, vs = (bf16_cuda(np.ascontiguousarray(x[seqs][:, hs, step:step + 1])) for x, hs in ((qd, qh), (kd, heads), (vd, heads)))
            module.decode(qs, e["pool"], d["unit_base"], d["unit_tab"], d["unit_flags"], d["tmeta"], d["segments"],
                          d["cta_segments"], d["unit_slots"], e["kstat"], e["vstat"], e["tail_k"], e["tail_v"], ks, vs, cache.step,
                          qs, e["pm"], e["pl"], e["po"], e["prompt"], SCALE, 1)
            module.decode_merge(qs, e["pm"], e["pl"], e["po"], 0, d["unit_slots"], e["kstat"], e["vstat"], e["tail_k"], e["tail_v"],
                                ks, vs, cache.step, qs, SCALE, gather=gather.arguments())
        fulls = [gather.wait().float().cpu().numpy()[:, :, 0] for _, gather, _, _, _ in parts]      # then the consumers
        for cache, _, _, _, _ in parts:
            cache.advance()
        assert all((f == fulls[0]).all() for f in fulls)
        outs.append(fulls[0])
    module.check_device_error()
    assert all(int(gather.seen.item()) == 3 and gather.sync.tolist() == [0, 3] for _, gather, _, _, _ in parts)
    assert_fp_close(np.stack(outs, 1), whole, f"units sharded over {len(shards)} parts, outputs gathered by peer stores")
