"""KV-cache write path (rotate + quantise + pack) against the CPU oracle and the reference extension."""
import numpy as np
import pytest
import torch

import triattention_oracle as orc
from ref_harness import RefRunner, ref_logical
import layouts
from triattention_b200.kernels.prefill import F16, I4, I8, Q4, Prefill
from triattention_b200.maps import INF
from util import bf16_cuda, code_mismatch, make_inputs, ulp_diff

pytestmark = pytest.mark.gpu

# Allowance of the IEEE oracle against fast-math kernels: approximate division moves a scale by a few
# ulp, which flips a code only where x*inv sits on a rounding boundary.
SCALE_ULP, CODE_RATE = 4, 2e-3


def run_write(module, q, k, v, want4=True):
    """Product write path on [B,H,T,128] inputs (float32 numpy holding bf16 values, or bf16 CUDA tensors); returns
    logical numpy arrays per batch."""
    b, hq, t, _ = q.shape
    hk, tiles = k.shape[1], (t + 63) // 64
    pre = Prefill(module, None)
    formats = frozenset({F16, I8, I4})
    ops = pre.operands(b, hq, hk, t, want4, want4, formats, "cuda")
    qd, kd, vd = (x if torch.is_tensor(x) else bf16_cuda(x) for x in (q, k, v))
    module.prepare_qk(qd, kd, ops["q8"], ops["qa"], ops["k8"], ops["ka"], ops["partial"], ops["kstat"], ops["q4x"],
                      ops["qa4"], ops["k4x"], ops["ka4"], ops["k4"])
    module.pack_v(vd, ops["partial"], ops["vstat"], ops["v16"], ops["v8"], ops["v4"], ops["v8h"])
    torch.cuda.synchronize()
    cpu = lambda x: x.detach().cpu().numpy()
    blob = lambda x, n: cpu(x).reshape(b, hk, tiles, n)
    res = dict(q8=cpu(ops["q8"]).reshape(b, hq, t, 128), qa=cpu(ops["qa"]).reshape(b, hq, t),
               k8=layouts.unpack_k8(blob(ops["k8"], 8192)), ka=cpu(ops["ka"]).reshape(b, hk, tiles, 4),
               kstat=cpu(ops["kstat"]).reshape(b, hk, 3, 128), vstat=cpu(ops["vstat"]).reshape(b, hk, 3, 128),
               v16=layouts.unpack_v16(blob(ops["v16"], 16384)), v8=layouts.unpack_v8(blob(ops["v8"], 8192)),
               v4=layouts.unpack_v4(blob(ops["v4"], 4096)))
    # the fp16 rendering of the INT8 codes (the tensor-core operand of the prefill) holds exactly the codes
    v8h = layouts.unpack_v16(blob(ops["v8h"], 16384))
    assert (v8h.astype(np.float32) == res["v8"].astype(np.float32)).all()
    if want4:
        res.update(q4=cpu(ops["q4x"]).reshape(b, hq, t, 128), qa4=cpu(ops["qa4"]).reshape(b, hq, t),
                   k4x=layouts.unpack_k8(blob(ops["k4x"], 8192)), k4=layouts.unpack_k4(blob(ops["k4"], 4096)),
                   ka4=cpu(ops["ka4"]).reshape(b, hk, tiles, 4))
    return res


def oracle_write(q, k, v):
    q8, qa, q4, qa4 = orc.quantize_q(q)
    kstat = orc.channel_stats(k)
    k8, ka, k4, ka4 = orc.quantize_k(k, kstat[:, 0])
    vstat = orc.channel_stats(v)
    v16, v8, v4 = orc.pack_v(v, vstat)
    return dict(q8=q8, qa=qa, q4=q4, qa4=qa4, kstat=kstat, k8=k8, ka=ka, k4=k4, ka4=ka4, vstat=vstat, v16=v16, v8=v8, v4=v4)


@pytest.mark.parametrize("hq,hk,t,batch", [(4, 2, 200, 2), (8, 2, 512, 1), (2, 1, 1, 1), (2, 1, 63, 1), (2, 2, 64, 1),
                                           (2, 1, 65, 1), (3, 1, 129, 1), (24, 8, 1024, 1)])
def test_write_vs_oracle(module, hq, hk, t, batch):
    q, k, v = make_inputs(hq, hk, t, seed=11, batch=batch)
    got = run_write(module, q, k, v)
    worst = {}
    for b in range(batch):
        want = oracle_write(q[b], k[b], v[b])
        assert ulp_diff(got["kstat"][b][:, 0], want["kstat"][:, 0]).max() <= SCALE_ULP
        for name in ("qa", "qa4", "ka", "ka4"):
            assert ulp_diff(got[name][b], want[name]).max() <= SCALE_ULP, name
        assert ulp_diff(got["vstat"][b], want["vstat"]).max() <= SCALE_ULP
        for name in ("q8", "q4", "k8", "k4", "v8", "v4"):
            rate, big = code_mismatch(got[name][b], want[name])
            worst[name] = max(worst.get(name, 0.0), rate)
            assert big <= 1 and rate <= CODE_RATE, (name, rate, big)
        assert (got["k4x"][b] == got["k4"][b]).all()          # the packed and widened INT4 K codes are the same codes
        d16 = np.abs(got["v16"][b].astype(np.float32) - want["v16"].astype(np.float32))
        assert (d16 <= np.abs(want["v16"].astype(np.float32)) * 2.0 ** -10 + 1e-6).all()
    print("code mismatch rates vs IEEE oracle", worst)


def assert_write_equals_reference(got, b, o):
    """Every code and every scale / statistic bit pattern of sequence b of a product write (run_write) equals what the
    reference extension left in its operand buffers `o` (RefRunner.prefill) for the same sequence."""
    ref = ref_logical(o)
    compared = []
    for name in ("qa", "ka", "qa4", "ka4"):
        if name in ref:
            assert (got[name][b].view(np.uint32) == ref[name].view(np.uint32)).all(), name
            compared.append(name)
    assert (got["kstat"][b][:, 0].view(np.uint32) == ref["kstat"][:, 0].view(np.uint32)).all()
    assert (got["vstat"][b].view(np.uint32) == ref["vstat"].view(np.uint32)).all()
    for name in ("q8", "q4", "k8", "k4", "v8", "v4"):
        if name in ref:
            assert (got[name][b] == ref[name]).all(), (name, code_mismatch(got[name][b], ref[name]))
            compared.append(name)
    assert (got["v16"][b].view(np.uint16) == ref["v16"].view(np.uint16)).all()
    return compared


@pytest.mark.parametrize("hq,hk,t", [(4, 2, 200), (8, 2, 512), (2, 1, 65), (24, 8, 1024)])
def test_write_bit_exact_vs_reference(module, ref_ext, hq, hk, t):
    """Codes and scale bit patterns equal the reference kernels' on the same GPU."""
    q, k, v = make_inputs(hq, hk, t, seed=23, batch=2)
    got = run_write(module, q, k, v)
    run = RefRunner(ref_ext)
    bands = np.array([[2, 3]] * hq, np.int64) if t > 128 else np.array([[1, INF]] * hq, np.int64)
    for b in range(2):
        o = run.prefill(bf16_cuda(q[b])[None], bf16_cuda(k[b])[None], bf16_cuda(v[b])[None], bands, 0.088, with_decode=True)
        torch.cuda.synchronize()
        assert_write_equals_reference(got, b, o)


def test_write_strided_inputs(module):
    """The HF hook hands over [B,T,H,128] storage viewed as [B,H,T,128]."""
    q, k, v = make_inputs(4, 2, 130, seed=5, batch=2)
    base = run_write(module, q, k, v)
    pre = Prefill(module, None)
    ops = pre.operands(2, 4, 2, 130, True, True, frozenset({F16, I8, I4}), "cuda")
    tr = lambda x: bf16_cuda(x).transpose(1, 2).contiguous().transpose(1, 2)
    module.prepare_qk(tr(q), tr(k), ops["q8"], ops["qa"], ops["k8"], ops["ka"], ops["partial"], ops["kstat"], ops["q4x"],
                      ops["qa4"], ops["k4x"], ops["ka4"], ops["k4"])
    module.pack_v(tr(v), ops["partial"], ops["vstat"], ops["v16"], ops["v8"], ops["v4"])
    torch.cuda.synchronize()
    assert (ops["q8"].cpu().numpy().reshape(2, 4, 130, 128) == base["q8"]).all()
    assert (layouts.unpack_k8(ops["k8"].cpu().numpy().reshape(2, 2, 3, 8192)) == base["k8"]).all()
    assert (layouts.unpack_v8(ops["v8"].cpu().numpy().reshape(2, 2, 3, 8192)) == base["v8"]).all()


def test_argument_errors(module):
    q = torch.zeros((1, 2, 8, 128), dtype=torch.float16, device="cuda")
    with pytest.raises(RuntimeError):
        module.prepare_qk(q, q, q, q, q, q, q, q)


@pytest.mark.parametrize("rows", [64, 100])
def test_requantize_with_given_statistics(module, rows):
    """tri_requantize_kv: rows that arrive after the prompt, quantised with the prompt's statistics, give the
    codes and scales the oracle's quantize_k / pack_v give for the same statistics (rows beyond the count are zero)."""
    hq, hk, t, batch = 4, 2, 300, 2
    q, k, v = make_inputs(hq, hk, t, seed=37, batch=batch)
    _, kn, vn = make_inputs(hq, hk, rows, seed=38, batch=batch)
    vn = vn * 1.7                                   # some values leave the prompt's range and are clamped
    ops = Prefill(module, None).operands(batch, hq, hk, t, False, False, frozenset({F16, I8}), "cuda")
    module.prepare_qk(bf16_cuda(q), bf16_cuda(k), ops["q8"], ops["qa"], ops["k8"], ops["ka"], ops["partial"], ops["kstat"])
    module.pack_v(bf16_cuda(v), ops["partial"], ops["vstat"], ops["v16"], ops["v8"], None, ops["v8h"])
    tiles = (rows + 63) // 64
    k8 = torch.empty((batch * hk, tiles, 8192), dtype=torch.uint8, device="cuda")
    v8 = torch.empty_like(k8)
    ka = torch.empty((batch * hk, tiles, 4), dtype=torch.float32, device="cuda")
    stats = ops["kstat"].clone(), ops["vstat"].clone()
    module.requantize_kv(bf16_cuda(kn), bf16_cuda(vn), ops["kstat"], ops["vstat"], k8, ka, v8)
    torch.cuda.synchronize()
    assert torch.equal(stats[0], ops["kstat"]) and torch.equal(stats[1], ops["vstat"])      # read only
    cpu = lambda x: x.detach().cpu().numpy()
    got_k = layouts.unpack_k8(cpu(k8).reshape(batch, hk, tiles, 8192))
    got_v = layouts.unpack_v8(cpu(v8).reshape(batch, hk, tiles, 8192))
    got_ka = cpu(ka).reshape(batch, hk, tiles, 4)
    kstat, vstat = cpu(ops["kstat"]).reshape(batch, hk, 3, 128), cpu(ops["vstat"]).reshape(batch, hk, 3, 128)
    for b in range(batch):
        want_k, want_ka, _, _ = orc.quantize_k(kn[b], kstat[b][:, 0])
        _, want_v, _ = orc.pack_v(orc.to_bf16(vn[b]), vstat[b])
        assert ulp_diff(got_ka[b], want_ka).max() <= SCALE_ULP
        for name, got, want in (("k8", got_k[b], want_k), ("v8", got_v[b], want_v)):
            rate, big = code_mismatch(got, want)
            assert big <= 1 and rate <= CODE_RATE, (name, rate, big)
        assert np.abs(got_v[b]).max() == 127 and not got_k[b].reshape(hk, -1, 128)[:, rows:].any()


def test_q_modes_skip_what_the_attention_does_not_read(module):
    """q_modes: a head without an INT4 band gets no INT4 codes, an un-quantised head no codes at all; what is written
    equals the unmasked run, and the prefill result does not change."""
    from triattention_b200.kernels.prefill import BandTable
    hq, hk, t = 6, 3, 200
    q, k, v = make_inputs(hq, hk, t, seed=43, batch=2)
    full = run_write(module, q, k, v)
    bands = np.asarray([[INF, INF]] * 2 + [[1, INF]] * 2 + [[INF, INF]] * 2, np.int64)
    table = BandTable.build(bands, (t + 63) // 64, hk, "cuda", bf16_kv=(2,))
    assert table.q_modes.tolist() == [1, 1, 3, 3, 0, 0]
    ops = Prefill(module, None).operands(2, hq, hk, t, True, True, frozenset({F16, I8, I4}), "cuda")
    for name in ("q8", "q4x"):
        ops[name].fill_(-128)
    ops["qa"].fill_(-1.0), ops["qa4"].fill_(-1.0)
    module.prepare_qk(bf16_cuda(q), bf16_cuda(k), ops["q8"], ops["qa"], ops["k8"], ops["ka"], ops["partial"], ops["kstat"],
                      ops["q4x"], ops["qa4"], ops["k4x"], ops["ka4"], ops["k4"], q_modes=table.q_modes)
    torch.cuda.synchronize()
    q8, q4 = ops["q8"].cpu().numpy().reshape(2, hq, t, 128), ops["q4x"].cpu().numpy().reshape(2, hq, t, 128)
    qa, qa4 = ops["qa"].cpu().numpy().reshape(2, hq, t), ops["qa4"].cpu().numpy().reshape(2, hq, t)
    assert (q8[:, :4] == full["q8"][:, :4]).all() and (qa[:, :4] == full["qa"][:, :4]).all()
    assert (q4[:, 2:4] == full["q4"][:, 2:4]).all() and (qa4[:, 2:4] == full["qa4"][:, 2:4]).all()
    assert (q8[:, 4:] == -128).all() and (qa[:, 4:] == -1).all()                    # un-quantised heads: untouched
    assert (q4[:, :2] == -128).all() and (q4[:, 4:] == -128).all() and (qa4[:, :2] == -1).all()


@pytest.mark.parametrize("case", ["all-formats", "int8-only", "identity-v", "raw-head-and-modes"])
def test_fused_write_equals_the_two_calls(module, case):
    """tri_write_kv (Q, K and V chains side by side on three streams) leaves byte for byte what prepare_qk followed by
    pack_v leave, and the caller's stream sees the finished buffers: copies queued right behind the call, on a stream of
    the caller's, are compared."""
    b, hq, hk, t = 2, 4, 2, 777
    q, k, v = (bf16_cuda(x) for x in make_inputs(hq, hk, t, seed=31, batch=b))
    int4 = case in ("all-formats", "raw-head-and-modes")
    formats = frozenset({F16}) if case == "identity-v" else frozenset({F16, I8, I4} if int4 else {F16, I8})
    q_modes = raw = None
    if case == "raw-head-and-modes":
        q_modes = torch.tensor([1, 3, 0, 2], dtype=torch.int32, device="cuda")
        raw = torch.tensor([0, 1], dtype=torch.int32, device="cuda")
    names = ("q8", "qa", "k8", "ka", "kstat", "vstat", "q4x", "qa4", "k4x", "ka4", "k4", "v16", "v8", "v4", "v8h")

    def fresh():
        ops = Prefill(module, None).operands(b, hq, hk, t, int4, int4, formats, "cuda")
        for name in names:
            if ops[name] is not None:
                ops[name].view(torch.uint8).fill_(0x5a)     # rows the modes leave untouched stay as they were in both
        return ops

    two = fresh()
    module.prepare_qk(q, k, two["q8"], two["qa"], two["k8"], two["ka"], two["partial"], two["kstat"], two["q4x"], two["qa4"],
                      two["k4x"], two["ka4"], two["k4"], q_modes=q_modes)
    module.pack_v(v, two["partial"], two["vstat"], two["v16"], two["v8"], two["v4"], two["v8h"], raw_heads=raw)
    want = {n: two[n].clone() for n in names if two[n] is not None}
    one = fresh()
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        for _ in range(3):      # repeated calls reuse the library's side streams and events
            module.write_kv(q, k, v, one["q8"], one["qa"], one["k8"], one["ka"], one["partial"], one["kstat"], one["partial_v"],
                            one["vstat"], one["q4x"], one["qa4"], one["k4x"], one["ka4"], one["k4"], q_modes=q_modes,
                            v16=one["v16"], v8=one["v8"], v4=one["v4"], v8h=one["v8h"], raw_heads=raw)
        got = {n: one[n].clone() for n in want}
    stream.synchronize()
    for n in want:
        assert torch.equal(got[n].view(torch.uint8), want[n].view(torch.uint8)), n
    with pytest.raises(RuntimeError):       # the two statistics passes run at the same time: one scratch buffer each
        module.write_kv(q, k, v, one["q8"], one["qa"], one["k8"], one["ka"], one["partial"], one["kstat"], one["partial"],
                        one["vstat"], one["q4x"], one["qa4"], one["k4x"], one["ka4"], one["k4"], v16=one["v16"], v8=one["v8"],
                        v4=one["v4"], v8h=one["v8h"])
