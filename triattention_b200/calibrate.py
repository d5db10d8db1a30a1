"""``python -m triattention_b200.calibrate`` — per-head error of every distance-band configuration.

Flags, grid, error measure and the ``triattention-calibration-v1`` output record are those of the reference's tool
(``triattention/calibrate.py:13-73``).  The cost differs: the reference runs one full prefill per grid point and layer
(86 KV-cache writes and 86 attention launches over every query row, of which it keeps the last ``--rows``); here a
layer is ONE KV-cache write and ONE attention launch that evaluates every grid point on the same operands and only
the query blocks holding the wanted rows (``Prefill.sweep`` -> ``tri_attention_sweep``).
"""
from __future__ import annotations

import argparse
import json
from pathlib import Path

import torch

from triattention_b200.maps import INF

W8 = (1, 2, 4, 8, 16, 32, 64, 128, 256, 512, INF)
W4 = (2, 4, 8, 16, 32, 64, 128, 256, 512, 1024, 2048, INF)


def grid():
    """The reference's grid (calibrate.py:17-18): for every INT8 distance the INT4 distances not below it, the INT8
    distance itself included; "never INT8" pairs only with "never INT4"."""
    points = []
    for w8 in W8:
        candidates = (INF,) if w8 == INF else sorted(set(W4) | {w8})
        points += [(w8, w4) for w4 in candidates if w4 >= w8]
    return points


def load_samples(path, tokenizer, response_tokens):
    """One JSON record per line with "prompt" and "response" (calibrate.py:21-28): the chat-rendered prompt followed by
    at most ``response_tokens`` tokens of the response.  Returns [(token ids, response length)]."""
    from triattention_b200.models import render_prompt

    def encode(text):
        return tokenizer(text, add_special_tokens=False).input_ids

    out = []
    with open(path) as lines:
        for record in map(json.loads, filter(str.strip, lines)):
            tail = encode(record["response"])[:response_tokens]
            out.append((encode(render_prompt(tokenizer, record["prompt"])) + tail, len(tail)))
    return out


def head_errors(outputs, exact, weight, chunk=8):
    """The reference's error measure (calibrate.py:53-62) for all configurations at once.  outputs [C,H,R,128] (any
    float type), exact [H,R,128] float32, weight = the layer's output projection [hidden, H*128].  Per head and
    configuration: delta^T (W_h^T W_h) delta summed over the rows, divided by the energy of the exact projected output.
    Returns float64 [H, C] on the CPU."""
    heads = exact.shape[0]
    w = weight.float()
    per_head = w.view(w.shape[0], heads, 128).permute(1, 0, 2)
    gram = per_head.transpose(1, 2) @ per_head
    energy = float((exact.transpose(0, 1).reshape(-1, heads * 128) @ w.T).square().sum())
    parts = []
    for c0 in range(0, outputs.shape[0], chunk):        # bounded temporary: a few configurations at a time
        delta = outputs[c0:c0 + chunk].float() - exact[None]
        parts.append(torch.einsum("chtd,hde,chte->ch", delta, gram, delta))
    return (torch.cat(parts).double().cpu() / energy).transpose(0, 1).contiguous()


class Calibration:
    """Accumulates the error table layer by layer; ``attention`` is the hook body installed into the model."""

    def __init__(self, executor, configs, rows):
        self.executor, self.configs, self.rows, self.errors = executor, configs, rows, {}

    def attention(self, mod, query, key, value, scaling):
        from triattention_b200.models import exact_attention
        heads, t = query.shape[1], query.shape[2]
        ref = exact_attention(query, key, value, scaling)
        outputs, row0 = self.executor.sweep(self.configs, query, key, value, scaling, rows=self.rows)
        first = max(0, t - self.rows)
        table = head_errors(outputs[:, 0, :, first - row0:], ref[0, :, first:].float(), mod.o_proj.weight)
        if mod.layer_idx not in self.errors:
            self.errors[mod.layer_idx] = torch.zeros(heads, len(self.configs), dtype=torch.float64)
        self.errors[mod.layer_idx] += table
        return ref

    def record(self, model_type, samples):
        return dict(format="triattention-calibration-v1", model_type=model_type, rows=self.rows, samples=samples,
                    configs=self.configs,
                    errors={layer: (e / samples).tolist() for layer, e in sorted(self.errors.items())})


@torch.inference_mode()
def main() -> None:
    from triattention_b200.kernels.extension import load_extension
    from triattention_b200.kernels.prefill import Prefill
    from triattention_b200.maps import uniform
    from triattention_b200.models import load_model, load_tokenizer, use_attention
    parser = argparse.ArgumentParser(description="Measure the per-head error of every distance-band configuration.")
    parser.add_argument("--model", required=True)
    parser.add_argument("--samples", required=True)
    parser.add_argument("--output", required=True)
    parser.add_argument("--rows", type=int, default=1024)
    parser.add_argument("--response-tokens", type=int, default=256)
    args = parser.parse_args()
    tokenizer, model = load_tokenizer(args.model), load_model(args.model)
    samples = load_samples(args.samples, tokenizer, args.response_tokens)
    run = Calibration(Prefill(load_extension(), uniform(INF, INF)), grid(), args.rows)
    use_attention(model, "triattention_calibration", run.attention)
    for n, (ids, _) in enumerate(samples, 1):
        model(input_ids=torch.tensor([ids], device="cuda"), use_cache=False, logits_to_keep=1)
        print(f"sample {n}/{len(samples)}: {len(ids)} tokens", flush=True)
    Path(args.output).write_text(json.dumps(run.record(model.config.model_type, len(samples))))


if __name__ == "__main__":
    main()
