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
timed region); roofline = algorithmic cache bytes per launch / CUDA-event time of the split-KV kernel
against the measured HBM copy peak; cpu_baseline = the CPU oracle port on a bounded sample.
`--impl reference` times that CPU port alone (the reference has no CPU or sm_100 implementation of its
own to run; its CUDA extension is used only as the parity oracle in the tests).
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


def kv_kinds(seed=1):
    return [str(x) for x in np.random.default_rng(seed).permutation(np.array(CONFIG["kinds"]))]


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

    def summary(self):
        rows = [r for r in self.rows if len(r) == 6 and r[0].isdigit()]
        if not rows:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=[], samples=0)
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in rows)]
        return dict(sm_mhz=float(np.median([int(r[0]) for r in rows])), sm_max_mhz=float(rows[0][1]), reasons=reasons,
                    samples=len(rows))


def build_cache(batch, seed0, tile_costs=None, fused_merge=False, part=None, split_group=None):
    """Synthetic prompt K/V -> quantised cache through the product's write kernels.  Returns (cache, plan).
    part = sequences written per pass (None = all at once); with it the prompts are generated on the GPU."""
    from triattention_b200.kernels.decode import DecodeCache
    from triattention_b200.kernels.extension import load_extension
    from triattention_b200.kernels.prefill import Prefill
    from triattention_b200.maps import per_kv_head
    hq, hk, t = CONFIG["heads_q"], CONFIG["heads_kv"], CONFIG["cache_tokens"]
    module = load_extension()
    cache = DecodeCache(module, max_tail=256, fused_merge=fused_merge, split_group=split_group,
                        **({"tile_costs": tile_costs} if tile_costs else {}))
    pre = Prefill(module, per_kv_head(kv_kinds(), hq // hk), cache)
    make = synth_cuda if part else (lambda shape, seed: synth(shape, seed).cuda())
    step = part or batch
    k = torch.empty((step, hk, t, 128), dtype=torch.bfloat16, device="cuda")
    v = torch.empty_like(k)
    q = torch.zeros((1, 1, 1, 128), dtype=torch.bfloat16, device="cuda").expand(step, hq, t, 128)   # Q does not enter the cache
    for first in range(0, batch, step):
        n = min(step, batch - first)
        for b in range(n):
            k[b] = make((hk, t, 128), 2 * (seed0 + first + b))
            v[b] = make((hk, t, 128), 2 * (seed0 + first + b) + 1)
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


def run_prefill(args):
    """Secondary metric: INT8 TOP/s of the banded prefill (benchmark configuration 3: 28 Q / 4 KV heads, batch 2,
    16384 tokens, 3 INT8 + 1 INT4 KV heads) including the fused KV-cache write.  One GPU, one JSON line."""
    from triattention_b200.kernels.extension import load_extension
    from triattention_b200.kernels.prefill import Prefill
    from triattention_b200.maps import per_kv_head
    torch.cuda.set_device(0)
    module = load_extension()
    b, hq, hk, t = args.batch, 28, 4, args.tokens
    kinds = [str(x) for x in np.random.default_rng(1).permutation(np.array(["int8", "int8", "int8", "int4"]))]
    q = torch.stack([synth((hq, t, 128), 10 + i) for i in range(b)]).cuda()
    k = torch.stack([synth((hk, t, 128), 20 + i) for i in range(b)]).cuda()
    v = torch.stack([synth((hk, t, 128), 30 + i) for i in range(b)]).cuda()
    pre = Prefill(module, per_kv_head(kinds, hq // hk))
    scale = 128 ** -0.5
    warmup = warm_up(lambda: pre(0, q, k, v, scale), max(3, args.warmup))
    module.check_device_error()
    steps = max(1, min(args.steps, 20))
    with ClockSampler(0) as clocks:
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
    print(json.dumps(dict(metric="prefill_int8_tops", value=ops / (ms_all / 1e3) / 1e12, unit="TOP/s", n_gpus=1, steps=steps,
                          warmup=warmup, ms_per_step=ms_all, higher_is_better=True, dtype="int8 (QK^T) / fp16 (P.V)", data="synthetic",
                          config=dict(workload=f"prefill C3: 28 Q / 4 KV heads, batch {b}, {t} tokens, map {kinds}, incl. KV write",
                                      l2="operands larger than L2"),
                          roofline=dict(bound="tensor", achieved=tops, peak=nominal, unit="TOP/s", frac=tops / nominal,
                                        kernel="prefill_kernel", ms_per_launch=ms_all - ms_write, ops_per_launch=ops,
                                        peak_source="nominal dense INT8 (2 x bf16 nominal); no measured INT8 peak in MEASURED_PEAKS.json",
                                        traffic=None),
                          kv_write_ms=ms_write, kv_write_bytes=write_bytes, kv_write_gbs=write_bytes / (ms_write / 1e3) / 1e9,
                          kv_write_frac_of_measured_hbm=write_bytes / (ms_write / 1e3) / 1e9 / peak_hbm()[0],
                          clocks=dict(clocks.summary(), untimed_steps_of_the_same_load_added_for_sampling=extra))))


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

    names = ("prepare_qk", "pack_v", "attention", "cache_store", "cache_store_bf16", "decode")
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
                          decode_tokens_per_s_cuda_graph=batch * (new - 1) / graph_s,
                          decode_tokens_per_s_layer_by_layer=batch * (new - 1) / eager_s,
                          decode_loop_s=dict(cuda_graph=graph_s, layer_by_layer=eager_s),
                          time_inside_the_attention_library=library, clocks=clocks.summary())))


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
    warmup = max(3, args.warmup)
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
    warmup = warm_up(lambda: cache(0, qd, kd, vd, scale, out=out), max(warmup, 300) if split else warmup,
                     seconds=0.0 if split else 0.3)
    module.check_device_error()
    with ClockSampler(local) as clocks:
        ms_total = timed(lambda i: cache(0, qd, kd, vd, scale, out=out), args.steps, dist)
        ms_kernel = timed(lambda i: cache(0, qd, kd, vd, scale, phases=1, out=out), args.steps, dist)
        ms_stream = timed(lambda i: cache(0, qd, kd, vd, scale, phases=5, out=out), args.steps, dist)

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
            if not split and not (len(clocks.rows) < 8 and time.time() - t_extra < 4.0):
                break
            for i in range(200):
                cache(0, qd, kd, vd, scale, out=out)
            torch.cuda.synchronize()
            extra += 200
        if not torch.equal(out_host, out.cpu()):
            raise RuntimeError("e2e output differs from the device-resident run")
    module.check_device_error()
    if rank != 0:
        dist.destroy_process_group()
        return
    tokens = batch if split else batch * world
    peak, peak_kind = peak_hbm()
    bytes_per_launch = plan["payload_bytes"]
    kernel_s = ms_kernel / args.steps / 1e3
    achieved = bytes_per_launch / kernel_s / 1e9
    line = dict(metric="decode_tokens_per_s", value=tokens * args.steps / (ms_total / 1e3), unit="tokens/s", n_gpus=world,
                steps=args.steps, warmup=warmup, ms_per_step=ms_total / args.steps, higher_is_better=True,
                scaling="strong" if split else "weak", vs_baseline=None, dtype="int8", data="synthetic", config=CONFIG,
                e2e=dict(value=tokens * args.steps / (ms_e2e / 1e3), unit="tokens/s",
                         h2d_bytes_per_step=sum(x.numel() * 2 for x in host), d2h_bytes_per_step=out.numel() * 2),
                gpu_launches=(1 if cache.layers[0]["unit_done"] is not None else 2) * args.steps,
                roofline=dict(bound="hbm", achieved=achieved, peak=peak, unit="GB/s", frac=achieved / peak,
                              # ncu capture of a batch-8 case (profiles/decode_kernel_c2.md): reads = 1.0014 x algorithmic
                              # bytes, writes = 23.4 KB per segment; scaled by the tiles / segments of this launch
                              traffic=int(bytes_per_launch * 1.0014 + plan["segments"].shape[0] * 23400),
                              kernel="decode_kernel", us_per_launch=kernel_s * 1e6, bytes_per_launch=bytes_per_launch,
                              peak_source=f"{peak_kind} copy bandwidth", frac_of_8tbs=achieved / 8000.0,
                              copy_pipeline_only_gbs=bytes_per_launch / (ms_stream / args.steps / 1e3) / 1e9,
                              ctas=int(plan["cta_segments"].shape[0] - 1), segments=int(plan["segments"].shape[0])),
                hbm_gbs_whole_step=bytes_per_launch / (ms_total / args.steps / 1e3) / 1e9,
                clocks=dict(clocks.summary(), untimed_steps_of_the_same_load_added_for_sampling=extra))
    if split:
        line["sequence_split"] = f"every unit's tile range cut over {world} GPUs; one all-gather of folded partials per step"
    if batch != CONFIG["batch"]:
        line["reduced_case"] = f"batch {batch} instead of {CONFIG['batch']}: not a benchmark value"
    if args.cpu_steps > 0:
        line["cpu_baseline"] = CpuPort(os.cpu_count() or 1).run(args.cpu_steps, 1)[0]
    print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
