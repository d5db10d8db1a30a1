"""Task-table mode of the prefill attention (explicit tile lists per query block, four passes) against the CPU oracle
and the reference extension.  The reference has no caller for this mode; the tables here are random."""
import numpy as np
import pytest
import torch

import triattention_oracle as orc
from ref_harness import RefRunner
from triattention_b200.kernels.prefill import F16, I4, I8, Prefill
from util import assert_fp_close, bf16_cuda, make_inputs

pytestmark = pytest.mark.gpu
SCALE = 1.0 / np.sqrt(128.0)


def random_tables(hq, rows, seed):
    """Four tile lists per (head, block): [sink, diagonal] first, then random earlier tiles per pass; some blocks end a
    later pass with their diagonal tile (masked there), some name it in the middle of a list (not masked)."""
    rng = np.random.default_rng(seed)
    lists, groups, entries = {}, [0], []
    for h in range(hq):
        for qb in range(rows):
            earlier = np.arange(1, qb)
            pick = lambda p: sorted(rng.choice(earlier, size=rng.integers(0, len(earlier) + 1), replace=False).tolist()) if len(earlier) else []
            four = [[0] if qb == 0 else [0, qb], pick(0), pick(1), pick(2)]
            kind = rng.integers(0, 4)
            if qb > 0 and kind == 1:
                four[0], four[1] = [0], four[1] + [qb]            # diagonal masked at the end of the INT8 pass
            elif qb > 0 and kind == 2:
                four[0], four[3] = [0], four[3] + [qb]            # ... of the INT4-score pass
            elif qb > 1 and kind == 3:
                four[2] = [qb] + four[2] + [1]                     # diagonal in the middle: not masked
            lists[(h, qb)] = four
            for one in four:
                entries += one
                groups.append(len(entries))
    return lists, np.asarray(groups, np.int32), np.asarray(entries + [0], np.int32)


def product_tasks(module, q, k, v, groups, entries):
    b, hq, t, _ = q.shape
    hk = k.shape[1]
    pre = Prefill(module, None)
    ops = pre.operands(b, hq, hk, t, True, False, frozenset({F16, I8, I4}), "cuda")
    module.prepare_qk(bf16_cuda(q), bf16_cuda(k), ops["q8"], ops["qa"], ops["k8"], ops["ka"], ops["partial"], ops["kstat"],
                      ops["q4x"], ops["qa4"], ops["k4x"], ops["ka4"])
    module.pack_v(bf16_cuda(v), ops["partial"], ops["vstat"], ops["v16"], ops["v8"], ops["v4"], None)
    out = torch.empty((b, t, hq, 128), dtype=torch.bfloat16, device="cuda").transpose(1, 2)
    module.attention_tasks(torch.from_numpy(groups).cuda(), torch.from_numpy(entries).cuda(), ops["v16"], ops["v8"], ops["v4"],
                           ops["vstat"], ops["q8"], ops["k8"], ops["qa"], ops["ka"], ops["q4x"], ops["k4x"], ops["qa4"],
                           ops["ka4"], out, SCALE, hk)
    module.check_device_error()
    return out.float().cpu().numpy()


def oracle_tasks(q, k, v, lists):
    hq, t, _ = q.shape
    hk, rows = k.shape[0], (t + 63) // 64
    _, o = orc.prefill(q, k, v, np.array([[orc.INF, orc.INF]] * hq), SCALE, return_operands=True)
    vstat = orc.channel_stats(v)
    v16, v8, v4 = orc.pack_v(v, vstat)
    sl2, pad = orc.sm_log2(SCALE), rows * 64 - t
    padq = lambda a: np.concatenate([a, np.zeros((hq, pad, 128), np.int8)], 1)
    pads = lambda a: np.concatenate([a * sl2, np.full((hq, pad), orc.FLT_MIN, np.float32)], 1).astype(np.float32)
    q8, q4, qs, qs4 = padq(o["q8"]), padq(o["q4"]), pads(o["qa"]), pads(o["qa4"])
    out = np.zeros((hq, rows * 64, 128), np.float32)
    for (h, qb), (t16, t8, t4v, tq4) in lists.items():
        kh, sl = h // (hq // hk), slice(qb * 64, (qb + 1) * 64)
        out[h, sl] = orc.prefill_block(q8[h, sl], qs[h, sl], o["k8"][kh], o["ka"][kh], v16[kh], v8[kh], vstat[kh], t, qb,
                                       t16, t8, tq4, q4[h, sl], qs4[h, sl], o["k4"][kh], o["ka4"][kh], tiles_i4=t4v, v4=v4[kh])
    return out[:, :t]


@pytest.mark.parametrize("hq,hk,t", [(4, 2, 330), (2, 1, 512), (3, 1, 65)])
def test_tasks_vs_oracle(module, hq, hk, t):
    q, k, v = make_inputs(hq, hk, t, seed=91, batch=2)
    lists, groups, entries = random_tables(hq, (t + 63) // 64, seed=t)
    got = product_tasks(module, q, k, v, groups, entries)
    for b in range(2):
        assert_fp_close(got[b], orc.to_bf16(oracle_tasks(q[b], k[b], v[b], lists)), f"task tables, b={b}")


@pytest.mark.parametrize("hq,hk,t", [(4, 2, 330), (2, 1, 512)])
def test_tasks_vs_reference(module, ref_ext, hq, hk, t):
    q, k, v = make_inputs(hq, hk, t, seed=92, batch=1)
    lists, groups, entries = random_tables(hq, (t + 63) // 64, seed=7 * t)
    got = product_tasks(module, q, k, v, groups, entries)
    ref = RefRunner(ref_ext).prefill_tasks(bf16_cuda(q), bf16_cuda(k), bf16_cuda(v), groups, entries, SCALE)
    assert_fp_close(got[0], ref.float().cpu().numpy()[0], "task tables vs the reference kernel")


def test_bad_tile_number_is_reported(module):
    q, k, v = make_inputs(2, 1, 130, seed=93, batch=1)
    lists, groups, entries = random_tables(2, 3, seed=1)
    entries = entries.copy()
    entries[1] = 9                                  # the prompt has 3 tiles
    with pytest.raises(RuntimeError):
        product_tasks(module, q, k, v, groups, entries)
    module.error_word("cuda").zero_()
