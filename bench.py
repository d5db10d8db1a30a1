"""Benchmark of the quantised-attention decode path (benchmark configuration 2) on N B200s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

A step is one decode step of one attention layer for the whole batch: Llama-3.2-3B-shaped layer
(24 Q heads, 8 KV heads, head_dim 128), batch 32, one new token per sequence over a quantised KV cache of
8192 tokens; map = seeded per-KV-head assignment, 4 INT8 / 2 INT4 / 2 BF16.  The cache is written by the
product's own KV-write kernels from synthetic K/V (N(0,1) in bf16 with 1 % of the channels scaled x20).
Under torchrun every rank runs the same per-GPU workload on its own sequences (weak scaling; units are
independent, so there is no data-path collective).

Printed JSON (one line, rank 0): value = tokens/s with all inputs resident in HBM; e2e = the same through
the public DecodeCache call with host buffers (pinned H2D of q/k/v and D2H of the output inside the
timed region); roofline = algorithmic cache bytes per launch / CUDA-event time of the split-KV kernel (its own timed
region of max(steps, 100) launches) against the measured HBM copy peak; cpu_baseline = the CPU oracle port on a bounded sample.
After that timed region, outside it, the same line gets secondary records (each can be skipped with --no-extras):
  prefill     configuration 3 (28 Q / 4 KV heads, batch 2, 16384 tokens): INT8 TOP/s of the prefill kernel against the
              nominal dense INT8 peak and against i8_peak, and the KV-cache write in GB/s            (1 GPU runs)
  calibration the reference's calibration grid (86 uniform maps) on one layer in one pass (Prefill.sweep) against one full
              prefill per grid point, the loop of the reference's tool                               (1 GPU runs)
  long_tail   the benchmark's decode step with 16, 64 and 256 rows in the BF16 tail of generated tokens (--tail-rows N
              measures the whole line at one such length)                                           (1 GPU runs)
  i8_peak     what back-to-back tcgen05 kind::i8 MMAs (M128 N256 K32, operands in shared memory) sustain on this GPU
  ref_ext     the reference's own CUDA extension (its sm_80 source compiled for sm_100, what a B200 runs today) timed
              on the same inputs: decode as 32 sequential batch-1 calls, prefill as 2 calls           (1 GPU runs)
  sharded_c5  configuration 5 (32 Q / 8 KV heads, 64 sequences x 131072 cached tokens) placed on the N GPUs by byte
              cost (sharding.shard_grid), each rank holding only its own units' cache, one decode step including the
              all-gather of the outputs; efficiency against the same step on one GPU, measured in the same run
  split       4 sequences x 131072 tokens with every unit's tile range cut over the N GPUs (fold in the split pass, one
              NCCL all-gather of (m, l, o) triples, strided merge) against one GPU                     (N > 1 runs)
`--impl reference` times the CPU port alone (the reference has no CPU implementation of its own to run; its CUDA
extension is timed in the ref_ext record above and is the parity oracle of the tests).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

INF = 1 << 20
CONFIG = dict(workload="decode C2: 24 Q / 8 KV heads, head_dim 128, batch 32, cache 8192 tokens, one layer-step",
              heads_q=24, heads_kv=8, batch=32, cache_tokens=8192, map="seed 1: 4 INT8 / 2 INT4 / 2 BF16 KV heads",
              l2="inputs larger than L2 (551 MB of cache per step per GPU)")
CONFIG["kinds"] = ["int8"] * 4 + ["int4"] * 2 + ["bf16"] * 2
# benchmark configuration 5 (--workload decode-long): a secondary line, same metric
CONFIG_LONG = dict(workload="decode C5: 32 Q / 8 KV heads, head_dim 128, batch 64, cache 131072 tokens, one layer-step",
                   heads_q=32, heads_kv=8, batch=64, cache_tokens=131072, map="seed 1: 4 INT4 / 3 INT8 / 1 BF16 KV heads",
                   l2="inputs larger than L2 (13.47 GB of cache per step per GPU)",
                   kinds=["int4"] * 4 + ["int8"] * 3 + ["bf16"])
FALLBACK_HBM_GBS = 6650.0


def kv_kinds(seed=1, cfg=None):
    return [str(x) for x in np.random.default_rng(seed).permutation(np.array((cfg or CONFIG)["kinds"]))]


def unit_kv(b, h, t, which):
    """K (which = 0) or V (1) of one (sequence, KV head) unit of the long workload, generated on the GPU from a seed
    of its own, so that a unit holds the same values whichever GPU it is placed on: N(0,1) with one of the 128
    channels (1 %) scaled x20."""
    return synth_cuda((1, t, 128), 2 * (b * 64 + h) + which)[0]


def synth_cuda(shape, seed, fraction=0.01, factor=20.0):
    """synth() generated on the GPU (the long workload's prompts are 270 M values per sequence)."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(shape, generator=g, device="cuda", dtype=torch.float32)
    h = shape[0]
    pick = torch.randperm(h * 128, generator=g, device="cuda")[: int(round(fraction * h * 128))]
    scale = torch.ones(h * 128, device="cuda")
    scale[pick] = factor
    return (x * scale.view(h, 1, 128)).to(torch.bfloat16)


def synth(shape, seed, fraction=0.01, factor=20.0):
    """N(0,1) [H,T,128] with round(fraction*H*128) channels scaled by `factor` for all tokens; bf16."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(shape, generator=g, dtype=torch.float32)
    h = shape[0]
    pick = torch.randperm(h * 128, generator=g)[: int(round(fraction * h * 128))]
    x.view(h, -1, 128)[pick // 128, :, pick % 128] *= factor
    return x.to(torch.bfloat16)


def peak_hbm():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()   # the exact child started above
            self.proc.wait()
            self.thread.join(timeout=2)

    def mark(self):
        """Samples taken before this call (the warm-up) are left out of the summary."""
        self.first = len(self.rows)

    def summary(self):
        rows = [r for r in self.rows[getattr(self, "first", 0):] if len(r) == 6 and r[0].isdigit()]
        if not rows:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=[], samples=0)
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in rows)]
        return dict(sm_mhz=float(np.median([int(r[0]) for r in rows])), sm_max_mhz=float(rows[0][1]), reasons=reasons,
                    samples=len(rows))


def build_cache(batch, seed0, tile_costs=None, fused_merge=False, part=None, split_group=None, cfg=None, heads=None,
                sequences=None, exchange="nccl"):
    """Synthetic prompt K/V -> quantised cache through the product's write kernels.  Returns (module, cache, plan).
    part = sequences written per pass (None = all at once); with it the prompts are generated on the GPU.
    cfg = the configuration (default: the benchmark's); heads / sequences = the KV heads and sequence numbers this
    GPU holds (unit sharding; with them every unit is generated from its own seed, see unit_kv)."""
    from triattention_b200 import sharding
    from triattention_b200.kernels.decode import DecodeCache
    from triattention_b200.kernels.extension import load_extension
    from triattention_b200.kernels.prefill import Prefill
    from triattention_b200.maps import per_kv_head
    cfg = cfg or CONFIG
    hq, hk, t = cfg["heads_q"], cfg["heads_kv"], cfg["cache_tokens"]
    g = hq // hk
    module = load_extension()
    cache = DecodeCache(module, max_tail=256, fused_merge=fused_merge, split_group=split_group, exchange=exchange,
                        **({"tile_costs": tile_costs} if tile_costs else {}))
    fn = per_kv_head(kv_kinds(cfg=cfg), g)
    by_unit = heads is not None
    if by_unit:
        shard = sharding.Shard(0, slice(0, batch), tuple(heads))
        fn = sharding.slice_map(fn, shard, g, hq)
        hk, hq = len(heads), len(heads) * g
    sequences = list(range(seed0, seed0 + batch)) if sequences is None else list(sequences)
    pre = Prefill(module, fn, cache)
    make = synth_cuda if part else (lambda shape, seed: synth(shape, seed).cuda())
    step = part or batch
    k = torch.empty((step, hk, t, 128), dtype=torch.bfloat16, device="cuda")
    v = torch.empty_like(k)
    q = torch.zeros((1, 1, 1, 128), dtype=torch.bfloat16, device="cuda").expand(step, hq, t, 128)   # Q does not enter the cache
    for first in range(0, batch, step):
        n = min(step, batch - first)
        for b in range(n):
            if by_unit:
                for i, h in enumerate(heads):
                    k[b, i], v[b, i] = unit_kv(sequences[first + b], h, t, 0), unit_kv(sequences[first + b], h, t, 1)
            else:
                k[b] = make((hk, t, 128), 2 * sequences[first + b])
                v[b] = make((hk, t, 128), 2 * sequences[first + b] + 1)
        table, ops = pre.write(0, q[:n], k[:n], v[:n])
        cache.store(0, t, ops, table.host, k[:n], v[:n], table.bf16_kv, first_sequence=first, sequences=batch)
    torch.cuda.synchronize()
    pre.buffers.clear(), pre.views.clear()
    del k, v, ops
    torch.cuda.empty_cache()
    return module, cache, cache.layers[0]["plan"]


def warm_up(step, at_least, seconds=0.3):
    """Untimed warm-up: at least `at_least` steps, and on until `seconds` of load have passed (SM clocks ramp over the
    first tenth of a second).  Returns the number of steps run."""
    done, t0 = 0, time.time()
    while done < at_least or time.time() - t0 < seconds:
        step()
        done += 1
        if done % 16 == 0:
            torch.cuda.synchronize()
    torch.cuda.synchronize()
    return done


def timed(fn, steps, dist, finish=None):
    """`steps` calls of fn between barriers + synchronize; CUDA events; max over ranks.  Returns ms.
    finish() runs before the stop event: it joins side streams into the timed one."""
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    start.record()
    for i in range(steps):
        fn(i)
    if finish is not None:
        finish()
    stop.record()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    ms = torch.tensor([start.elapsed_time(stop)], device="cuda")
    if dist is not None:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return float(ms.item())


class CpuPort:
    """The CPU oracle port on one sequence of the workload: one decode step of 24 heads over 8192 cached tokens."""
    def __init__(self, threads):
        self.SAMPLE = (f"1 of the {CONFIG['batch']} sequences per step, one layer-step ({CONFIG['heads_q']} heads over "
                       f"{CONFIG['cache_tokens']} cached tokens); numpy/IEEE restatement of the reference's CUDA arithmetic")
        sys.path.insert(0, str(ROOT / "oracle"))
        import triattention_oracle as orc
        self.orc, self.threads = orc, threads
        torch.set_num_threads(threads)
        hq, hk, t = CONFIG["heads_q"], CONFIG["heads_kv"], CONFIG["cache_tokens"]
        self.kinds, self.g = kv_kinds(), hq // hk
        self.k, self.v = synth((hk, t, 128), 0).float().numpy(), synth((hk, t, 128), 1).float().numpy()
        self.bands = np.array([[1, INF] if kind == "int4" else [INF, INF] for kind in self.kinds for _ in range(self.g)], np.int64)
        kstat = orc.channel_stats(self.k)
        k8, ka, k4, ka4 = orc.quantize_k(self.k, kstat[:, 0])
        vstat = orc.channel_stats(self.v)
        v16, v8, v4 = orc.pack_v(self.v, vstat)
        self.ops = dict(kstat=kstat, k8=k8, ka=ka, k4=k4, ka4=ka4, vstat=vstat, v16=v16, v8=v8, v4=v4)
        self.qd = synth((hq, 1, 128), 7).float().numpy()[:, 0]
        self.kc, self.vc = synth((hk, 1, 128), 8).float().numpy()[:, 0], synth((hk, 1, 128), 9).float().numpy()[:, 0]

    def step(self):
        orc, hk, t = self.orc, CONFIG["heads_kv"], CONFIG["cache_tokens"]
        tk, tv = np.zeros((hk, 4, 128), np.float32), np.zeros((hk, 4, 128), np.float32)
        out = orc.decode_step(self.qd, self.ops, self.bands, t, 128 ** -0.5, tk, tv, self.kc, self.vc, 0, 4, None)
        for kh, kind in enumerate(self.kinds):     # BF16 heads: exact attention over the raw prompt
            if kind == "bf16":
                kk, vv = np.concatenate([self.k[kh], self.kc[kh][None]]), np.concatenate([self.v[kh], self.vc[kh][None]])
                for h in range(kh * self.g, (kh + 1) * self.g):
                    out[h] = orc.exact_decode(self.qd[h], kk, vv, 128 ** -0.5)
        return out

    def run(self, steps, warmup):
        for _ in range(warmup):
            self.step()
        t0 = time.perf_counter()
        for _ in range(steps):
            out = self.step()
        seconds = time.perf_counter() - t0
        assert np.isfinite(out).all()
        return dict(value=steps / seconds, unit="tokens/s", cores=self.threads, kind="port", sample=self.SAMPLE), seconds


def run_reference(args, rank):
    if rank != 0:
        return
    base, seconds = CpuPort(os.cpu_count() or 1).run(args.steps, args.warmup)
    line = dict(metric="decode_tokens_per_s", value=base["value"], unit="tokens/s", n_gpus=args.gpus, steps=args.steps,
                warmup=args.warmup, ms_per_step=seconds * 1e3 / args.steps, higher_is_better=True, scaling="weak",
                vs_baseline=None, dtype="int8", data="synthetic", config=CONFIG, impl="reference", cpu_baseline=base,
                e2e=dict(value=base["value"], unit="tokens/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0),
                note="the reference has no CPU path and no sm_100 kernel; this arm times the CPU oracle port of its arithmetic")
    print(json.dumps(line))


def measure_i8_peak(seconds=0.1):
    """Back-to-back tcgen05 kind::i8 MMAs (M128 N256 K32, operands resident in shared memory), one CTA per SM, timed
    with CUDA events: the INT8 tensor throughput this GPU sustains when it does nothing else (tests/probe/i8_peak.cu)."""
    import ctypes
    sys.path.insert(0, str(ROOT / "tests"))
    try:
        from probe import build_probe
        lib = build_probe.load()
    except (ImportError, OSError, FileNotFoundError) as e:
        return dict(unavailable=f"probe library not built: {e}")
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    err, ops = torch.zeros(1, dtype=torch.int32, device="cuda"), ctypes.c_int64()
    stream = torch.cuda.current_stream().cuda_stream

    def run(iterations):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        if lib.tri_i8_peak(sms, iterations, ctypes.byref(ops), err.data_ptr(), stream) != 0:
            raise RuntimeError(lib.tri_probe_last_error().decode())
        stop.record()
        torch.cuda.synchronize()
        return start.elapsed_time(stop)

    run(2000)
    ms = run(20000)                                        # sizes the long run
    iterations = int(min(1 << 22, max(20000, 20000 * seconds * 1e3 / ms)))
    with ClockSampler(0) as clocks:
        ms = min(run(iterations) for _ in range(2))
        per_cta = ops.value                                # of the timed launch (every launch overwrites it)
        run(iterations * 4)                                # the same load a little longer, for the clock sampler
    if int(err.item()):
        return dict(unavailable="the peak kernel's bounded wait ran out")
    tops = sms * per_cta / (ms / 1e3) / 1e12
    return dict(tops=tops, ms=ms, mma="tcgen05.mma kind::i8 M128 N256 K32, A and B in shared memory", ctas=sms,
                mmas_per_cta=4 * iterations, nominal_tops=4500.0, frac_of_nominal=tops / 4500.0, clocks=clocks.summary())


def prefill_inputs(b, hq, hk, t):
    kinds = [str(x) for x in np.random.default_rng(1).permutation(np.array(["int8", "int8", "int8", "int4"]))]
    q = torch.stack([synth_cuda((hq, t, 128), 10 + i) for i in range(b)])
    k = torch.stack([synth_cuda((hk, t, 128), 20 + i) for i in range(b)])
    v = torch.stack([synth_cuda((hk, t, 128), 30 + i) for i in range(b)])
    return kinds, q, k, v


def measure_prefill(b, t, steps, warmup, peak=None):
    """INT8 TOP/s of the banded prefill (benchmark configuration 3: 28 Q / 4 KV heads, batch 2, 16384 tokens, 3 INT8 +
    1 INT4 KV heads) and the KV-cache write in GB/s.  One GPU."""
    from triattention_b200.kernels.extension import load_extension
    from triattention_b200.kernels.prefill import Prefill
    from triattention_b200.maps import per_kv_head
    module = load_extension()
    hq, hk = 28, 4
    kinds, q, k, v = prefill_inputs(b, hq, hk, t)
    pre = Prefill(module, per_kv_head(kinds, hq // hk))
    scale = 128 ** -0.5
    ran = warm_up(lambda: pre(0, q, k, v, scale), max(3, warmup))
    module.check_device_error()
    steps = max(1, min(steps, 20))
    with ClockSampler(torch.cuda.current_device()) as clocks:
        ms_all = timed(lambda i: pre(0, q, k, v, scale), steps, None) / steps
        ms_write = timed(lambda i: pre.write(0, q, k, v), steps, None) / steps
        t_extra, extra = time.time(), 0
        while len(clocks.rows) < 8 and time.time() - t_extra < 4.0:   # same load, untimed, until nvidia-smi has sampled it
            pre(0, q, k, v, scale)
            torch.cuda.synchronize()
            extra += 1
    module.check_device_error()
    # KV-write traffic: Q once, K and V twice (statistics pass + quantising pass), every operand buffer written once
    # (Q codes only for the heads whose band needs them: BandTable.q_modes)
    table, written = pre.write(0, q, k, v)
    modes = table.q_modes.cpu()
    share = dict(q8=float((modes & 1).ne(0).float().mean()), q4x=float((modes & 2).ne(0).float().mean()))
    share.update(qa=share["q8"], qa4=share["q4x"])
    write_bytes = q.nbytes + 2 * k.nbytes + 2 * v.nbytes + int(sum(x.nbytes * share.get(name, 1.0) for name, x in written.items()
                                                                     if x is not None and name != "partial"))
    rows = (t + 63) // 64
    ops = b * hq * (rows * (rows + 1) // 2) * 2 * 64 * 64 * 128 * 2
    tops = ops / ((ms_all - ms_write) / 1e3) / 1e12
    nominal = 4500.0
    roofline = dict(bound="tensor", achieved=tops, peak=nominal, unit="TOP/s", frac=tops / nominal, kernel="prefill_kernel",
                    ms_per_launch=ms_all - ms_write, ops_per_launch=ops, peak_source="nominal dense INT8 (2 x bf16 nominal)",
                    traffic=None)
    if peak and "tops" in peak:
        roofline.update(measured_i8_tops=peak["tops"], frac_of_measured_i8=tops / peak["tops"])
    pre.buffers.clear(), pre.views.clear()
    return dict(metric="prefill_int8_tops", value=ops / (ms_all / 1e3) / 1e12, unit="TOP/s", steps=steps, warmup=warmup,
                warmup_steps_run=ran, ms_per_step=ms_all, dtype="int8 (QK^T) / fp16 high + low parts (P.V)",
                config=dict(workload=f"prefill C3: 28 Q / 4 KV heads, batch {b}, {t} tokens, map {kinds}, incl. KV write",
                            l2="operands larger than L2"),
                roofline=roofline, kv_write_ms=ms_write, kv_write_bytes=write_bytes,
                kv_write_gbs=write_bytes / (ms_write / 1e3) / 1e9,
                kv_write_frac_of_measured_hbm=write_bytes / (ms_write / 1e3) / 1e9 / peak_hbm()[0],
                clocks=dict(clocks.summary(), untimed_steps_of_the_same_load_added_for_sampling=extra))


def measure_calibration(steps, t=8192, rows=1024):
    """One layer of the calibration grid (86 uniform maps, 32 Q / 8 KV heads, batch 1, the last `rows` of `t` query rows kept):
    all grid points in one KV-cache write and one attention launch (Prefill.sweep) against the reference tool's loop of one
    full prefill per grid point (calibrate.py:46-63 of the reference), both on this library's kernels.  One GPU."""
    from triattention_b200.calibrate import grid
    from triattention_b200.kernels.extension import load_extension
    from triattention_b200.kernels.prefill import Prefill
    from triattention_b200.maps import INF, uniform
    module, configs, scale = load_extension(), grid(), 128 ** -0.5
    _, q, k, v = prefill_inputs(1, 32, 8, t)
    one = Prefill(module, uniform(INF, INF))
    shared, loop = {}, []
    for w8, w4 in configs:
        loop.append(Prefill(module, uniform(w8, w4)))
        loop[-1].buffers = shared
    first = t - rows

    def per_point():
        return [pre(0, q, k, v, scale)[0, :, first:] for pre in loop]

    warm_up(lambda: one.sweep(configs, q, k, v, scale, rows=rows), 3)
    per_point()
    module.check_device_error()
    steps = max(1, min(steps, 10))
    ms_sweep = timed(lambda i: one.sweep(configs, q, k, v, scale, rows=rows), steps, None) / steps
    ms_loop = timed(lambda i: per_point(), 2, None) / 2
    out, row0 = one.sweep(configs, q, k, v, scale, rows=rows)
    same = sum(bool(torch.equal(out[c, 0, :, first - row0:], ref)) for c, ref in enumerate(per_point()))
    module.check_device_error()
    del out
    one.buffers.clear(), one.views.clear(), shared.clear()
    return dict(metric="calibration_grid_points_per_s", value=len(configs) / (ms_sweep / 1e3), unit="grid points/s (one layer)",
                ms_per_layer=ms_sweep, ms_per_layer_one_prefill_per_point=ms_loop, speedup=ms_loop / ms_sweep,
                grid_points=len(configs), grid_points_bit_equal_to_their_own_run=same, steps=steps,
                config=dict(workload=f"calibration grid, 32 Q / 8 KV heads, batch 1, {t} tokens, last {rows} rows kept"))


def run_prefill(args):
    """--workload prefill: the prefill record alone, as its own JSON line."""
    torch.cuda.set_device(0)
    peak = measure_i8_peak()
    line = measure_prefill(args.batch, args.tokens, args.steps, args.warmup, peak)
    line.update(n_gpus=1, higher_is_better=True, data="synthetic", i8_peak=peak)
    print(json.dumps(line))


def measure_ref_ext(steps):
    """The kernel to beat: the reference's own CUDA extension (its sm_80 source compiled for sm_100, which is what its
    loader runs on a B200, kernels/extension.py:23-25,45), driven like its Python executors drive it, on this
    benchmark's inputs.  The reference is batch 1, so the 32 sequences of a decode step are 32 calls one after the
    other and the 2 sequences of the prefill 2 calls; its kernels have no un-quantised head kind, so the BF16 KV heads
    of configuration 2 are INT8 heads here (fewer bytes than the product streams for them).  Baseline leg only."""
    sys.path.insert(0, str(ROOT / "oracle"))
    try:
        import build_ref
        from ref_harness import RefRunner
        run = RefRunner(build_ref.load())
    except (ImportError, OSError, FileNotFoundError) as e:
        return dict(unavailable=f"reference extension not built: {e}")
    scale = 128 ** -0.5
    out = dict(kernel="prefill_sm80.cu compiled with -gencode arch=compute_100,code=sm_100 (the reference's own flags)")
    # decode, configuration 2
    hq, hk, t, batch = CONFIG["heads_q"], CONFIG["heads_kv"], CONFIG["cache_tokens"], CONFIG["batch"]
    bands = np.array([[1, INF] if kind == "int4" else [INF, INF] for kind in kv_kinds() for _ in range(hq // hk)], np.int64)
    zero_q = torch.zeros((1, 1, 1, 128), dtype=torch.bfloat16, device="cuda").expand(1, hq, t, 128)
    states = []
    for b in range(batch):
        k, v = synth((hk, t, 128), 2 * b).cuda()[None], synth((hk, t, 128), 2 * b + 1).cuda()[None]
        o = run.prefill(zero_q, k, v, bands, scale, attention=False)
        states.append(run.decode_setup(o, bands, max_tail=256))
        del o
    qd, kd, vd = (torch.stack([synth((h, 1, 128), 100 + i + 1000 * b) for b in range(batch)]).cuda() for i, h in enumerate((hq, hk, hk)))
    step = lambda i: [run.decode(states[b], qd[b:b + 1], kd[b:b + 1], vd[b:b + 1], scale) for b in range(batch)]
    for i in range(3):
        step(i)
    ms = timed(step, steps, None) / steps
    out.update(decode_tokens_per_s=batch / (ms / 1e3), decode_ms_per_step=ms, decode_calls_per_step=batch,
               decode_splits_of_tiles=int(states[0]["per"]),
               decode_workload=f"{CONFIG['workload']}; BF16 KV heads run as INT8 heads; 32 sequential batch-1 calls")
    del states
    torch.cuda.empty_cache()
    # prefill, configuration 3
    hq, hk, t, b = 28, 4, 16384, 2
    kinds, q, k, v = prefill_inputs(b, hq, hk, t)
    bands = np.array([[1, INF] if kind == "int4" else [INF, INF] for kind in kinds for _ in range(hq // hk)], np.int64)
    call = lambda i: [run.prefill(q[j:j + 1], k[j:j + 1], v[j:j + 1], bands, scale, with_decode=True) for j in range(b)]
    call(0)
    reps = max(1, min(steps, 5))
    ms = timed(call, reps, None) / reps
    rows = (t + 63) // 64
    ops = b * hq * (rows * (rows + 1) // 2) * 2 * 64 * 64 * 128 * 2
    out.update(prefill_ms=ms, prefill_tops=ops / (ms / 1e3) / 1e12,
               prefill_workload=f"prefill C3: 28 Q / 4 KV heads, batch {b} as {b} calls, {t} tokens, map {kinds}, incl. its KV write")
    return out


def long_inputs(cfg, batch):
    """Decode-step inputs of the long workload for sequences 0 .. batch-1, the same on every rank."""
    hq, hk = cfg["heads_q"], cfg["heads_kv"]
    return [torch.stack([synth_cuda((h, 1, 128), 5000 + 10 * b + i) for b in range(batch)]) for i, h in enumerate((hq, hk, hk))]


def time_steps(step, steps, dist, warm=5):
    for i in range(warm):          # count-based: with a collective in the step every rank runs the same number
        step(i)
    torch.cuda.synchronize()
    return timed(step, steps, dist) / steps


def measure_sharded_c5(rank, world, dist, steps):
    """Configuration 5 (32 Q / 8 KV heads, 64 sequences x 131072 cached tokens, 4 INT4 / 3 INT8 / 1 BF16 KV heads) as
    ONE job on N GPUs: sharding.shard_grid places (batch slice) x (KV-head group) rectangles by the per-head cache
    bytes under the mixed map, every rank writes and holds only its own units' cache, and a step is the rank's decode
    plus the all-gather that gives every rank the whole output.  Strong scaling: efficiency = t(1 GPU) / (N x t(N)),
    the one-GPU time measured by rank 0 in this same run on the same data."""
    from triattention_b200 import sharding
    from triattention_b200.maps import per_kv_head
    cfg = CONFIG_LONG
    hq, hk, t, batch = cfg["heads_q"], cfg["heads_kv"], cfg["cache_tokens"], cfg["batch"]
    g, scale = hq // hk, 128 ** -0.5
    kinds = kv_kinds(cfg=cfg)
    fn = per_kv_head(kinds, g)
    costs = sharding.head_costs(fn(0, hq).numpy(), hk, t, fn.bf16_kv_heads(0))
    qd, kd, vd = long_inputs(cfg, batch)
    record = dict(workload=cfg["workload"], map=kinds, scaling="strong", head_cache_bytes_per_sequence=[int(c) for c in costs])
    one = None
    if rank == 0:
        module, cache, plan = build_cache(batch, 0, part=2, cfg=cfg, heads=list(range(hk)))
        out = torch.empty_like(qd)
        ms1 = time_steps(lambda i: cache(0, qd, kd, vd, scale, out=out), steps, None)
        module.check_device_error()
        one = dict(ms=ms1, out=out.clone(), bytes=int(plan["payload_bytes"]))
        record.update(one_gpu_ms_per_step=ms1, one_gpu_tokens_per_s=batch / (ms1 / 1e3),
                      one_gpu_gbs=one["bytes"] / (ms1 / 1e3) / 1e9, cache_bytes_per_step=one["bytes"])
        del cache, plan
        torch.cuda.empty_cache()
    if world == 1:
        record.update(n_gpus=1, tokens_per_s=record["one_gpu_tokens_per_s"], ms_per_step=record["one_gpu_ms_per_step"],
                      per_gpu_gbs=record["one_gpu_gbs"], efficiency=1.0, shards=[dict(sequences=[0, batch], kv_heads=list(range(hk)))])
        return record
    dist.barrier()
    shards = sharding.shard_grid(batch, costs, world)
    mine = shards[rank]
    heads, qh = list(mine.kv_heads), list(mine.q_heads(g))
    nb = mine.batch.stop - mine.batch.start
    module, cache, plan = build_cache(nb, 0, part=2, cfg=cfg, heads=heads, sequences=range(mine.batch.start, mine.batch.stop))
    take = lambda x, hs: x[mine.batch].index_select(1, torch.as_tensor(hs, device=x.device)).contiguous()
    ql, kl, vl = take(qd, qh), take(kd, heads), take(vd, heads)
    gather = sharding.OutputGatherer(shards, g, batch, hq, ql)
    out_local = gather.send            # the decode writes straight into the send slot of the gather (strided is fine)
    full = [None]

    def step(i):
        cache(0, ql, kl, vl, scale, out=out_local)
        full[0] = gather(out_local)

    ms_nccl = time_steps(step, steps, dist)
    ms_local = time_steps(lambda i: cache(0, ql, kl, vl, scale, out=out_local), steps, dist)
    module.check_device_error()
    # the same step with the gather fused into the merge kernel: output rows stored into every GPU's full tensor by peer
    # stores, a flag per rank and one bounded wait; no collective call
    ms_peer, peer_note = None, None
    try:
        peer = sharding.PeerOutputGatherer(module, shards, g, batch, hq, ql.device)

        def step_peer(i):
            full[0] = cache(0, ql, kl, vl, scale, gather=peer)

        ms_peer = time_steps(step_peer, steps, dist)
        module.check_device_error()
    except (RuntimeError, ImportError) as e:      # no symmetric memory on this system: every rank fails alike
        peer_note = str(e)[:200]
    ms = min(ms_nccl, ms_peer) if ms_peer is not None else ms_nccl
    loads = torch.tensor([float(plan["payload_bytes"])], device="cuda")
    every = [torch.zeros_like(loads) for _ in range(world)]
    dist.all_gather(every, loads)
    loads = [float(x.item()) for x in every]
    if rank == 0:
        diff = float((full[0].float() - one["out"].float()).abs().max())
        record.update(n_gpus=world, tokens_per_s=batch / (ms / 1e3), ms_per_step=ms, ms_per_step_without_the_output_gather=ms_local,
                      ms_per_step_gather_by_nccl=ms_nccl, ms_per_step_gather_by_peer_stores=ms_peer, peer_gather_unavailable=peer_note,
                      per_gpu_gbs=max(loads) / (ms / 1e3) / 1e9, bytes_per_rank_max=max(loads),
                      bytes_per_rank_mean=sum(loads) / world, balance_mean_over_max=sum(loads) / world / max(loads),
                      efficiency=one["ms"] / (world * ms), max_abs_diff_vs_one_gpu=diff,
                      output_gather="nccl: one all_gather_into_tensor of the bf16 outputs per step (the decode writes into the send slot; "
                                    "the gathered blocks are the output when the shards are equal batch slices); peer stores: the "
                                    "merge kernel writes every row into every GPU's full output tensor, one flag per rank, one "
                                    "bounded wait; ms_per_step is the faster of the two",
                      shards=[dict(sequences=[s.batch.start, s.batch.stop], kv_heads=list(s.kv_heads)) for s in shards])
    del cache, plan
    torch.cuda.empty_cache()
    return record


def measure_split(rank, world, dist, steps):
    """Long-context decode with fewer units than the GPUs can share out: 4 sequences x 131072 cached tokens of
    configuration 5's layer, every unit's kept-tile range cut into one cost-balanced part per GPU.  A step is this
    rank's split pass with the fold inside it, one NCCL all-gather of the (m, l, o) triples, and the merge that reads
    the gathered buffer in place.  Speed-up against the same 4 sequences whole on one GPU (rank 0, same run)."""
    cfg = dict(CONFIG_LONG, batch=4, workload="decode, sequence split: 32 Q / 8 KV heads, 4 sequences x 131072 cached tokens")
    hk, batch, scale = cfg["heads_kv"], cfg["batch"], 128 ** -0.5
    qd, kd, vd = long_inputs(cfg, batch)
    out = torch.empty_like(qd)
    record, one = dict(workload=cfg["workload"], scaling="strong"), None
    if rank == 0:
        module, cache, plan = build_cache(batch, 0, part=2, cfg=cfg, heads=list(range(hk)))
        ms1 = time_steps(lambda i: cache(0, qd, kd, vd, scale, out=out), steps, None, warm=50)
        module.check_device_error()
        one = dict(ms=ms1, out=out.clone())
        record.update(one_gpu_ms_per_step=ms1, cache_bytes_per_step=int(plan["payload_bytes"]))
        del cache, plan
        torch.cuda.empty_cache()
    dist.barrier()
    how = dict(nccl="fold inside the split pass; one all_gather_into_tensor (NCCL) of [units, 8, 130] f32 per rank; the merge "
                    "reads the gathered buffer by stride",
               peer="fold inside the split pass writes the triples, then a flag, into every GPU's exchange buffer by peer "
                    "stores over NVLink; the merge waits per unit for the flags; no collective call in the step")
    for exchange in ("nccl", "peer"):
        try:
            module, cache, plan = build_cache(batch, 0, part=2, cfg=cfg, heads=list(range(hk)), split_group=dist.group.WORLD,
                                              exchange=exchange)
        except (RuntimeError, ImportError) as e:       # no symmetric memory on this system: every rank fails alike
            if rank == 0:
                record[exchange] = dict(unavailable=str(e)[:200])
            continue
        ms = time_steps(lambda i: cache(0, qd, kd, vd, scale, out=out), steps, dist, warm=50)
        ms_local = time_steps(lambda i: cache(0, qd, kd, vd, scale, phases=1, out=out), steps, dist, warm=5)
        cache(0, qd, kd, vd, scale, out=out)
        module.check_device_error()
        if rank == 0:
            record[exchange] = dict(ms_per_step=ms, tokens_per_s=batch / (ms / 1e3), speedup_vs_one_gpu=one["ms"] / ms,
                                    efficiency=one["ms"] / (world * ms), ms_split_pass_alone=ms_local,
                                    rank0_cache_bytes=int(plan["payload_bytes"]),
                                    max_abs_diff_vs_one_gpu=float((out.float() - one["out"].float()).abs().max()),
                                    exchange=how[exchange])
        del cache, plan
        torch.cuda.empty_cache()
        dist.barrier()
    if rank == 0:
        best = max((r for r in (record.get("nccl"), record.get("peer")) if r and "ms_per_step" in r),
                   key=lambda r: r["speedup_vs_one_gpu"])
        record.update(n_gpus=world, ms_per_step=best["ms_per_step"], speedup_vs_one_gpu=best["speedup_vs_one_gpu"],
                      efficiency=best["efficiency"])
    return record


def run_model(args):
    """Secondary metric: benchmark configuration 4 end to end.  Random-init Llama-3.2-3B architecture (28 layers, hidden 3072,
    24 / 8 heads, head_dim 128, intermediate 8192 as in the public 3B configuration, vocab 128256), bf16 weights
    ~ N(0, 0.02); batch x prompt token ids uniform from a seed; greedy new tokens; per-layer seeded map of 5 INT8 /
    2 INT4 / 1 BF16 KV heads.  Prints tokens/s of the prompt pass and of the decode loop, layer-by-layer from Python
    and with the decode step captured in a CUDA graph."""
    from transformers import LlamaConfig, LlamaForCausalLM
    from triattention_b200.maps import INF, from_bands
    from triattention_b200.models import TriAttention
    torch.cuda.set_device(0)
    batch = args.batch
    prompt, new, layers, hq, hk = args.tokens if args.tokens != 16384 else 4096, args.new_tokens, 28, 24, 8
    cfg = LlamaConfig(hidden_size=3072, intermediate_size=8192, num_hidden_layers=layers, num_attention_heads=hq,
                      num_key_value_heads=hk, head_dim=128, vocab_size=128256, max_position_embeddings=prompt + new + 8,
                      rope_theta=500000.0, tie_word_embeddings=True)
    torch.manual_seed(0)
    with torch.device("cuda"):
        model = LlamaForCausalLM(cfg).to(torch.bfloat16).eval()
    for prm in model.parameters():
        prm.data.normal_(0.0, 0.02, generator=None)
    rng = np.random.default_rng(2)
    bands, bf16 = {}, {}
    for layer in range(layers):
        kinds = rng.permutation(np.array(["int8"] * 5 + ["int4"] * 2 + ["bf16"]))
        bands[str(layer)] = [[1, INF] if kind == "int4" else [INF, INF] for kind in kinds for _ in range(hq // hk)]
        bf16[str(layer)] = [i for i, kind in enumerate(kinds) if kind == "bf16"]
    engine = TriAttention(model, from_bands(bands, model, bf16), max_new_tokens=new + 1)
    ids = torch.randint(0, cfg.vocab_size, (batch, prompt), generator=torch.Generator().manual_seed(1)).cuda()

    def timed_generate(graph):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        with torch.inference_mode():
            model(input_ids=ids, use_cache=False, logits_to_keep=1)
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        rows = engine.generate(ids, new, eos=(), cuda_graph=graph)   # runs the prompt pass again, then the decode loop
        torch.cuda.synchronize()
        t2 = time.perf_counter()
        assert len(rows) == batch and all(len(r) == new for r in (rows if batch > 1 else [rows]))
        prefill_s = t1 - t0
        return prefill_s, (t2 - t1) - prefill_s

    # The very first prompt pass also plans every layer's cache on the host (28 distinct per-layer maps = 28 plans:
    # tile states, compaction, the cost-balanced cut, one table upload each); later prompts of this length reuse them.
    torch.cuda.synchronize()
    t_first = time.perf_counter()
    with torch.inference_mode():
        model(input_ids=ids, use_cache=False, logits_to_keep=1)
    torch.cuda.synchronize()
    first_prompt_s, planning_s = time.perf_counter() - t_first, engine.decode_cache.plan_seconds
    timed_generate(False)   # warm-up (library handles, caches, clocks)
    with ClockSampler(0) as clocks:
        prefill_s, eager_s = timed_generate(False)
        _, graph_s = timed_generate(True)
    engine.module.check_device_error()

    # Where the time goes: CUDA events around every call into the library during one more prompt pass and a few
    # layer-by-layer decode steps (everything else is the model's own GEMMs and element-wise kernels).
    spans = {}

    def watch(name):
        inner = getattr(engine.module, name)

        def call(*a, **k):
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record()
            result = inner(*a, **k)
            end.record()
            spans.setdefault(name, []).append((begin, end))
            return result
        setattr(engine.module, name, call)
        return inner

    names = ("write_kv", "attention", "cache_store", "cache_store_bf16", "decode")
    originals = {name: watch(name) for name in names}
    few = min(new, 9)
    engine.generate(ids, few, eos=())
    torch.cuda.synchronize()
    for name, inner in originals.items():
        setattr(engine.module, name, inner)
    ms = {name: sum(b.elapsed_time(e) for b, e in spans.get(name, [])) for name in names}
    prompt_ms = sum(ms[name] for name in names if name != "decode")
    library = dict(prompt_pass_ms=prompt_ms, prompt_pass_share=prompt_ms / (prefill_s * 1e3),
                   decode_ms_per_step=ms["decode"] / max(1, few - 1),
                   decode_share_of_graph_step=ms["decode"] / max(1, few - 1) / (graph_s * 1e3 / (new - 1)),
                   by_call_ms={k: round(v, 3) for k, v in ms.items()})
    print(json.dumps(dict(metric="generate_tokens_per_s", value=batch * (new - 1) / graph_s, unit="tokens/s", n_gpus=1,
                          higher_is_better=True, dtype="bf16 model, int8 / int4 / bf16 KV cache", data="synthetic",
                          config=dict(workload=f"end to end C4: random-init Llama-3.2-3B architecture, batch {batch} x {prompt} prompt "
                                               f"tokens, {new} greedy new tokens, per-layer map 5 INT8 / 2 INT4 / 1 BF16 KV heads"),
                          prompt_tokens_per_s=batch * prompt / prefill_s, prompt_pass_s=prefill_s,
                          host_planning=dict(seconds=planning_s, plans=len(engine.decode_cache.plans),
                                             share_of_a_prompt_pass=planning_s / prefill_s,
                                             first_prompt_pass_s_incl_planning_and_warmup=first_prompt_s,
                                             what="plan_streams + one table upload per layer, first prompt of a length only"),
                          decode_tokens_per_s_cuda_graph=batch * (new - 1) / graph_s,
                          decode_tokens_per_s_layer_by_layer=batch * (new - 1) / eager_s,
                          decode_loop_s=dict(cuda_graph=graph_s, layer_by_layer=eager_s),
                          time_inside_the_attention_library=library, clocks=clocks.summary())))


def grow_tail(cache, rows, qd, kd, vd, scale, out):
    """Decode steps with advance() until the next step's BF16 tail holds `rows` rows (the token it appends included)."""
    while cache.generated + 1 < rows:
        cache(0, qd, kd, vd, scale, out=out)
        cache.advance()


def measure_long_tail(cache, qd, kd, vd, scale, out, ms_one_row, lengths=(16, 64, 256), steps=100):
    """The benchmark's decode step later in a generation: the same cache, with 16, 64 and 256 rows in the BF16 tail of
    generated tokens instead of one (the merge kernel reads them exactly; above 8 rows the host picks its long-tail
    instantiation).  CUDA events over `steps` steps each; the tail is not advanced inside a timed region."""
    record = {"us_per_step_by_tail_rows": {"1": ms_one_row * 1e3}, "steps": steps, "workload": "decode C2, one layer-step"}
    for rows in lengths:
        grow_tail(cache, rows, qd, kd, vd, scale, out)
        warm_up(lambda: cache(0, qd, kd, vd, scale, out=out), 32, seconds=0.0)
        record["us_per_step_by_tail_rows"][str(rows)] = timed(lambda i: cache(0, qd, kd, vd, scale, out=out), steps, None) / steps * 1e3
    return record


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--workload", default="decode", choices=["decode", "decode-long", "prefill", "model"],
                        help="decode = the benchmark contract (benchmark configuration 2); decode-long = config 5 (64 sequences x "
                             "131072 cached tokens, 13.5 GB per step), prefill = config 3, model = config 4 end to end "
                             "through the Hugging Face hook: secondary metrics")
    parser.add_argument("--new-tokens", type=int, default=128, help="greedy new tokens of the model workload")
    parser.add_argument("--tokens", type=int, default=16384, help="prompt length of the prefill workload")
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=200)
    parser.add_argument("--warmup", type=int, default=10)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--cpu-steps", type=int, default=100,
                        help="timed steps of the CPU baseline leg (0 = skip); the default is about 10 s of CPU work")
    parser.add_argument("--tile-costs", default="", help="override the decode partition's cost model: bf16,k8v8,other (relative)")
    parser.add_argument("--fused-merge", action="store_true",
                        help="one launch per step: the CTA that finishes a unit's last segment merges it")
    parser.add_argument("--split", action="store_true",
                        help="with --gpus N: the SAME sequences on every GPU, every unit's tile range cut N ways (sequence "
                             "split, one all-gather of folded partials per step); strong scaling, a diagnostic")
    parser.add_argument("--tail-rows", type=int, default=1,
                        help="decode workloads: rows in the BF16 tail of generated tokens at the measured step (1..256; the "
                             "benchmark value is quoted at 1, the first generated token)")
    parser.add_argument("--no-extras", action="store_true",
                        help="skip the secondary records (prefill, i8_peak, ref_ext, sharded_c5, split) of the default workload")
    parser.add_argument("--batch", type=int, default=None,
                        help="sequences per GPU; anything but the configuration's is a reduced case for profiler captures, "
                             "flagged in the output")
    args = parser.parse_args()
    long_case = args.workload == "decode-long"
    if long_case:
        CONFIG.clear()
        CONFIG.update(CONFIG_LONG)
        if args.steps == 200:
            args.steps = 50
        if args.cpu_steps == 100:
            args.cpu_steps = 6      # one sequence-step of the CPU port over 131072 tokens takes two seconds
    if args.batch is None:
        args.batch = {"model": 16, "prefill": 2}.get(args.workload, CONFIG["batch"])
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if args.workload == "prefill":
        if rank == 0:
            run_prefill(args)
        return
    if args.workload == "model":
        if rank == 0:
            run_model(args)
        return
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        from datetime import timedelta
        # (a collective inside the step, --split, gets a short timeout: a rank that falls out of step then ends the run
        # within minutes)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local),
                                timeout=timedelta(seconds=120 if args.split else 600))
    hq, hk, batch = CONFIG["heads_q"], CONFIG["heads_kv"], args.batch
    costs = tuple(float(x) for x in args.tile_costs.split(",")) if args.tile_costs else None
    split = args.split and world > 1
    seed0 = 0 if split else rank * batch
    module, cache, plan = build_cache(batch, seed0=seed0, tile_costs=costs, fused_merge=args.fused_merge,
                                      part=2 if (long_case and not split) else None,
                                      split_group=dist.group.WORLD if split else None)
    scale = 128 ** -0.5
    # decode-step inputs: device-resident copies for `value`, pinned host copies for `e2e`
    host = [torch.stack([synth((h, 1, 128), 100 + i + 1000 * (seed0 + b)) for b in range(batch)]).pin_memory()
            for i, h in enumerate((hq, hk, hk))]
    qd, kd, vd = (x.cuda() for x in host)
    out = torch.empty_like(qd)
    out_host = torch.empty(out.shape, dtype=out.dtype).pin_memory()
    # With a collective inside the step every rank must run the same number of steps: no time-based loops then.
    # At least the requested warm-up steps (never fewer than 3), and on until the clocks have ramped: `warmup` in the
    # line is what was asked for, `warmup_steps_run` what actually ran.
    # The clock sampler (a child process) is started BEFORE the warm-up: starting it between the warm-up and the timed
    # region would leave the GPU idle for the milliseconds a fork takes, and the first timed steps would run on clocks
    # that had begun to drop (measured: 94.4 instead of 90.5 us per kernel launch over 20 timed steps).  Only the
    # samples taken from the start of the timed region on are summarised.
    if not 1 <= args.tail_rows <= cache.max_tail:
        raise SystemExit(f"--tail-rows must be in 1..{cache.max_tail}")
    grow_tail(cache, args.tail_rows, qd, kd, vd, scale, out)
    with ClockSampler(local) as clocks:
        warmup_run = warm_up(lambda: cache(0, qd, kd, vd, scale, out=out), max(3, args.warmup, 300 if split else 0),
                             seconds=0.0 if split else 0.3)
        module.check_device_error()
        if not split:   # (a few more steps behind the check's read-back, so that the timed region follows load, not a pause)
            warm_up(lambda: cache(0, qd, kd, vd, scale, out=out), 32, seconds=0.0)
        clocks.mark()
        ms_total = timed(lambda i: cache(0, qd, kd, vd, scale, out=out), args.steps, dist)
        # the kernel's average launch duration for the roofline: its own region of at least 100 launches, so that the
        # latency of the region's first launch does not weigh 5 % when few steps are asked for (`value` above is over
        # exactly the steps asked for)
        kernel_steps = max(args.steps, 100)
        ms_kernel = timed(lambda i: cache(0, qd, kd, vd, scale, phases=1, out=out), kernel_steps, dist)
        ms_stream = timed(lambda i: cache(0, qd, kd, vd, scale, phases=5, out=out), kernel_steps, dist)

        # e2e: host buffers in, host buffer out, every step; HostStepper rotates two sets of device buffers so
        # that the copies of neighbouring steps overlap this step's kernels
        from triattention_b200.kernels.decode import HostStepper
        stepper = HostStepper(cache, 0, qd.shape, kd.shape, qd.device)
        e2e_step = lambda i: stepper.submit(host[0], host[1], host[2], out_host, scale)
        for i in range(4):
            e2e_step(i)
        stepper.wait()
        ms_e2e = timed(e2e_step, args.steps, dist, finish=stepper.join)
        stepper.wait()
        # a short timed region gives nvidia-smi (100 ms period) little to sample: keep the same load running,
        # untimed, until a handful of samples are in
        t_extra, extra = time.time(), 0
        for burst in range(5 if split else 10 ** 6):
            if not split and not (len(clocks.rows) - clocks.first < 8 and time.time() - t_extra < 4.0):
                break
            for i in range(200):
                cache(0, qd, kd, vd, scale, out=out)
            torch.cuda.synchronize()
            extra += 200
        if not torch.equal(out_host, out.cpu()):
            raise RuntimeError("e2e output differs from the device-resident run")
    module.check_device_error()
    launches_per_step = 1 if cache.layers[0]["unit_done"] is not None else 2
    extras = {}
    if not args.no_extras and not long_case and not split and batch == CONFIG["batch"] and not args.fused_merge:
        # secondary records, outside the timed region of the benchmark value; the C2 cache is released first
        if world == 1 and args.tail_rows == 1:
            extras["long_tail"] = measure_long_tail(cache, qd, kd, vd, scale, out, ms_total / args.steps)
        del stepper, cache
        torch.cuda.empty_cache()
        extra_steps = max(5, min(args.steps, 20))
        if world == 1:
            extras["i8_peak"] = measure_i8_peak()
            extras["prefill"] = measure_prefill(2, 16384, extra_steps, 3, extras["i8_peak"])
            extras["ref_ext"] = measure_ref_ext(extra_steps)
            extras["calibration"] = measure_calibration(extra_steps)
            torch.cuda.empty_cache()
        extras["sharded_c5"] = measure_sharded_c5(rank, world, dist, extra_steps)
        if world > 1:
            extras["split"] = measure_split(rank, world, dist, extra_steps)
    if rank != 0:
        dist.destroy_process_group()
        return
    tokens = batch if split else batch * world
    peak, peak_kind = peak_hbm()
    bytes_per_launch = plan["payload_bytes"]
    kernel_s = ms_kernel / kernel_steps / 1e3
    achieved = bytes_per_launch / kernel_s / 1e9
    line = dict(metric="decode_tokens_per_s", value=tokens * args.steps / (ms_total / 1e3), unit="tokens/s", n_gpus=world,
                steps=args.steps, warmup=args.warmup, warmup_steps_run=warmup_run, ms_per_step=ms_total / args.steps,
                higher_is_better=True,
                scaling="strong" if split else "weak", vs_baseline=None, dtype="int8", data="synthetic", config=CONFIG,
                e2e=dict(value=tokens * args.steps / (ms_e2e / 1e3), unit="tokens/s",
                         h2d_bytes_per_step=sum(x.numel() * 2 for x in host), d2h_bytes_per_step=out.numel() * 2),
                gpu_launches=launches_per_step * args.steps,
                roofline=dict(bound="hbm", achieved=achieved, peak=peak, unit="GB/s", frac=achieved / peak,
                              # from an ncu capture of a batch-8 case: DRAM reads = 1.0014 x the algorithmic bytes, writes
                              # = 23.4 KB per segment; scaled to this launch by its tiles and segments
                              traffic=int(bytes_per_launch * 1.0014 + plan["segments"].shape[0] * 23400),
                              kernel="decode_kernel", us_per_launch=kernel_s * 1e6, bytes_per_launch=bytes_per_launch,
                              peak_source=f"{peak_kind} copy bandwidth", frac_of_8tbs=achieved / 8000.0,
                              copy_pipeline_only_gbs=bytes_per_launch / (ms_stream / kernel_steps / 1e3) / 1e9,
                              launches_timed=kernel_steps,
                              ctas=int(plan["cta_segments"].shape[0] - 1), segments=int(plan["segments"].shape[0])),
                hbm_gbs_whole_step=bytes_per_launch / (ms_total / args.steps / 1e3) / 1e9,
                clocks=dict(clocks.summary(), untimed_steps_of_the_same_load_added_for_sampling=extra))
    if split:
        line["sequence_split"] = f"every unit's tile range cut over {world} GPUs; one all-gather of folded partials per step"
    if args.tail_rows != 1:
        line["tail_rows"] = f"{args.tail_rows} rows in the BF16 tail instead of 1: not the benchmark value"
    if batch != CONFIG["batch"]:
        line["reduced_case"] = f"batch {batch} instead of {CONFIG['batch']}: not a benchmark value"
    line.update(extras)
    if args.cpu_steps > 0 and world == 1:
        line["cpu_baseline"] = CpuPort(os.cpu_count() or 1).run(args.cpu_steps, 1)[0]
    print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
