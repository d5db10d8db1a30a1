"""Record golden vectors from the reference's own CUDA extension (oracle/_ref) on a B200.

Run on the GPU box from the repository root:
    python tests/golden/make_golden.py <output directory>
and copy the produced ``*.npz`` into ``tests/golden/``.  Inputs are regenerated from seeds by
``triattention_oracle.synth`` (numpy, deterministic), so only the reference's outputs are stored.
"""
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent.parent.parent
for p in (ROOT / "oracle", ROOT / "tests"):
    sys.path.insert(0, str(p))
import build_ref  # noqa: E402
import triattention_oracle as orc  # noqa: E402
from ref_harness import RefRunner, bf16_cuda, ref_logical  # noqa: E402

INF = orc.INF
CASES = {
    # name: (Hq, Hkv, T, bands per Q head, outlier dims, outlier scale, row stride kept for big arrays)
    "small": (4, 2, 200, [[INF, INF], [INF, INF], [2, 3], [2, 3]], (7, 42, 77, 113), 4.0, 1),
    "c1": (8, 2, 512, [[INF, INF]] * 4 + [[1, INF]] * 4, (7, 42, 77, 113), 16.0, 4),
}


def inputs(name):
    hq, hk, t, bands, dims, scale, _ = CASES[name]
    seed = sum(name.encode())
    q = orc.synth((hq, t, 128), seed, outlier_dims=dims, outlier_scale=scale)
    k = orc.synth((hk, t, 128), seed + 1, outlier_dims=dims, outlier_scale=scale)
    v = orc.synth((hk, t, 128), seed + 2)
    qd = orc.synth((hq, 3, 128), seed + 3, outlier_dims=dims, outlier_scale=scale)
    kd = orc.synth((hk, 3, 128), seed + 4, outlier_dims=dims, outlier_scale=scale)
    vd = orc.synth((hk, 3, 128), seed + 5)
    return q, k, v, np.asarray(bands, np.int64), qd, kd, vd


def bf16_bits(t):
    return t.detach().contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def main(out_dir):
    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    run = RefRunner(build_ref.load())
    scale = 1.0 / np.sqrt(128.0)
    for name in CASES:
        hq, hk, t, _, _, _, keep = CASES[name]
        q, k, v, bands, qd, kd, vd = inputs(name)
        o = run.prefill(bf16_cuda(q)[None], bf16_cuda(k)[None], bf16_cuda(v)[None], bands, scale)
        lg = ref_logical(o)
        rec = {key: val for key, val in lg.items() if key in ("qa", "ka", "kstat", "vstat", "qa4", "ka4")}
        rec["q8"] = lg["q8"][:, ::keep]
        if "q4" in lg:
            rec["q4"] = lg["q4"][:, ::keep]
        for key in ("k8", "k4", "v8", "v4"):
            if key in lg:
                rec[key] = lg[key]
        rec["v16_bits"] = lg["v16"].view(np.uint16)[:, ::keep]
        rec["out_bits"] = bf16_bits(o["out"][0])[:, ::keep]
        # decode: three steps, two split sizes
        for per in (2, 1000):
            st = run.decode_setup(o, bands, max_tail=8, per=per)
            outs = []
            for step in range(3):
                od = run.decode(st, bf16_cuda(qd[:, step:step + 1])[None], bf16_cuda(kd[:, step:step + 1])[None],
                                bf16_cuda(vd[:, step:step + 1])[None], scale)
                outs.append(bf16_bits(od[0, :, 0]))
                st["step"].add_(1)
            rec[f"decode_bits_per{per}"] = np.stack(outs)
            if per == 2:
                rec["pm"], rec["pl"] = st["pm"].cpu().numpy(), st["pl"].cpu().numpy()
                rec["po"] = st["po"].cpu().numpy()
                rec["splits"] = np.int64(st["splits"])
        torch.cuda.synchronize()
        np.savez_compressed(out_dir / f"{name}.npz", **rec)
        print(name, {key: getattr(val, "shape", val) for key, val in rec.items()})


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else "golden_out")
