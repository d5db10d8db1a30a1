"""End to end through the Hugging Face hook: a small random-init Llama, batched prompts, greedy decode.
The reference's surface (TriAttention(model, map, n).generate) with its attention replaced by the sm_100a
kernels; logits are compared with the same model under exact attention."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def tiny_llama():
    from transformers import LlamaConfig, LlamaForCausalLM
    torch.manual_seed(0)
    cfg = LlamaConfig(hidden_size=512, intermediate_size=1024, num_hidden_layers=3, num_attention_heads=4,
                      num_key_value_heads=2, head_dim=128, vocab_size=1024, max_position_embeddings=1024,
                      rope_theta=500000.0)
    return LlamaForCausalLM(cfg).to(torch.bfloat16).cuda().eval()


@torch.inference_mode()
def test_generate_matches_exact_attention_logits():
    from triattention_b200.maps import INF, uniform
    from triattention_b200.models import TriAttention
    model = tiny_llama()
    ids = torch.randint(0, 1024, (3, 200), generator=torch.Generator().manual_seed(1)).cuda()
    model.set_attn_implementation("sdpa")
    ref = model(input_ids=ids, use_cache=True)
    ref_logits = ref.logits[:, -1].float()
    nxt = ref_logits.argmax(-1)
    ref2 = model(input_ids=nxt[:, None], past_key_values=ref.past_key_values, use_cache=True).logits[:, -1].float()

    engine = TriAttention(model, uniform(INF, INF), max_new_tokens=8)
    out = model(input_ids=ids, use_cache=False, logits_to_keep=1)
    got = out.logits[:, -1].float()
    assert all(engine.decode_cache.stored(layer) for layer in range(3))
    position = torch.full((3, 1), 200, device="cuda")
    got2 = model(input_ids=nxt[:, None], position_ids=position, use_cache=False).logits[:, -1].float()
    engine.module.check_device_error()
    for name, a, b in (("prefill", got, ref_logits), ("decode", got2, ref2)):
        cos = torch.nn.functional.cosine_similarity(a, b, dim=-1).min().item()
        rel = ((a - b).abs().max() / b.abs().max()).item()
        assert cos > 0.995 and rel < 0.1, (name, cos, rel)


@torch.inference_mode()
def test_generate_batched_and_single():
    from triattention_b200.maps import INF, per_kv_head
    from triattention_b200.models import TriAttention
    model = tiny_llama()
    engine = TriAttention(model, per_kv_head(["int8", "int4"], 2), max_new_tokens=6)
    ids = torch.randint(0, 1024, (2, 130), generator=torch.Generator().manual_seed(2)).cuda()
    rows = engine.generate(ids, 6, eos=())
    assert len(rows) == 2 and all(len(r) == 6 for r in rows)
    single = engine.generate(ids[:1], 6, eos=())
    assert isinstance(single, list) and len(single) == 6 and all(isinstance(t, int) for t in single)
    stop = engine.generate(ids[:1], 6, eos={single[2]})
    assert stop == single[:single.index(single[2])]


@torch.inference_mode()
def test_generate_cuda_graph_matches_eager():
    """One captured decode step replayed per token gives the same tokens as the layer-by-layer loop."""
    from triattention_b200.maps import per_kv_head
    from triattention_b200.models import TriAttention
    model = tiny_llama()
    engine = TriAttention(model, per_kv_head(["int8", "int4"], 2), max_new_tokens=12)
    ids = torch.randint(0, 1024, (3, 150), generator=torch.Generator().manual_seed(5)).cuda()
    eager = engine.generate(ids, 12, eos=())
    graph = engine.generate(ids, 12, eos=(), cuda_graph=True)
    assert graph == eager
    stop = eager[0][4]
    assert engine.generate(ids, 12, eos={stop}, cuda_graph=True) == engine.generate(ids, 12, eos={stop})
    # A longer generation is captured with the merge kernel for long tails (the short one above): same tokens again.
    longer = TriAttention(model, per_kv_head(["int8", "int4"], 2), max_new_tokens=24)
    assert longer.generate(ids, 24, eos=(), cuda_graph=True) == longer.generate(ids, 24, eos=())


@torch.inference_mode()
def test_generate_fold_tail_runs_past_the_tail():
    """fold_tail=True: the 64-row tail is folded into cached tiles twice on the way to 140 tokens.  Up to the first
    fold the tokens are those of the un-folded engine (same arithmetic); a captured graph is refused."""
    from triattention_b200.maps import per_kv_head
    from triattention_b200.models import TriAttention
    model = tiny_llama()
    ids = torch.randint(0, 1024, (2, 150), generator=torch.Generator().manual_seed(7)).cuda()
    plain = TriAttention(model, per_kv_head(["int8", "int4"], 2), max_new_tokens=140).generate(ids, 140, eos=())
    engine = TriAttention(model, per_kv_head(["int8", "int4"], 2), max_new_tokens=140, fold_tail=True)
    rows = engine.generate(ids, 140, eos=())
    assert all(len(r) == 140 for r in rows) and all(r[:65] == p[:65] for r, p in zip(rows, plain))
    assert all(engine.decode_cache.layers[layer]["extra"] == 2 for layer in range(3))
    assert engine.generate(ids, 140, eos=()) == rows          # a second prompt starts from a fresh cache
    with pytest.raises(RuntimeError):
        engine.generate(ids, 8, eos=(), cuda_graph=True)


class ReferenceEngine:
    """The reference's TriAttention (models.py:58-85 of the reference) restated over its own CUDA extension: the same
    Hugging Face hook, per layer its prepare_qk / pack_v / attention at the prompt and its decode afterwards, batch 1,
    greedy loop with use_cache=False.  Test infrastructure (the reference's Python package is not on the GPU box)."""

    def __init__(self, model, ref_ext, bands_fn, max_new_tokens):
        from ref_harness import RefRunner
        from triattention_b200.models import use_attention
        self.model, self.run, self.bands_fn, self.max_tail, self.layers = model, RefRunner(ref_ext), bands_fn, max_new_tokens, {}

        def attention(mod, query, key, value, scaling):
            layer = mod.layer_idx
            if query.shape[2] == 1 and layer in self.layers:
                return self.run.decode(self.layers[layer], query, key, value, scaling)
            bands = self.bands_fn(layer, query.shape[1]).numpy().astype(np.int64)
            o = self.run.prefill(query, key, value, bands, scaling)
            self.layers[layer] = self.run.decode_setup(o, bands, self.max_tail)
            return o["out"]

        use_attention(model, "reference_triattention", attention)

    @torch.inference_mode()
    def generate(self, ids, n):
        self.layers.clear()
        logits = self.model(input_ids=ids, use_cache=False, logits_to_keep=1).logits[:, -1].float()
        tokens, first = [], logits.clone()
        token = int(logits.argmax(-1))
        for i in range(n):
            tokens.append(token)
            if i + 1 == n:
                break
            position = torch.tensor([[ids.shape[1] + i]], device=ids.device)
            out = self.model(input_ids=torch.tensor([[token]], device=ids.device), position_ids=position, use_cache=False)
            for st in self.layers.values():
                st["step"].add_(1)
            token = int(out.logits[0, -1].argmax(-1))
        return first, tokens


@torch.inference_mode()
def test_hook_level_parity_with_the_reference_extension(ref_ext):
    """The whole surface at once: the same toy Llama run through the reference's kernels and through this library by
    way of the same attention hook (batch 1, the reference's limit): prompt-pass logits agree and the first 8 greedy
    tokens are the same."""
    from triattention_b200.maps import INF, from_bands
    from triattention_b200.models import TriAttention
    model = tiny_llama()
    bands = {str(layer): [[INF, INF], [INF, INF], [2, 3], [1, INF]] for layer in range(3)}
    fn = from_bands(bands, model)
    ids = torch.randint(0, 1024, (1, 330), generator=torch.Generator().manual_seed(11)).cuda()
    want_logits, want_tokens = ReferenceEngine(model, ref_ext, fn, 8).generate(ids, 8)
    engine = TriAttention(model, fn, max_new_tokens=8)
    got_logits = model(input_ids=ids, use_cache=False, logits_to_keep=1).logits[:, -1].float()
    got_tokens = engine.generate(ids, 8, eos=())
    engine.module.check_device_error()
    cos = torch.nn.functional.cosine_similarity(got_logits, want_logits, dim=-1).item()
    worst = (got_logits - want_logits).abs().max().item() / want_logits.abs().max().item()
    assert cos > 0.9999 and worst < 0.02, (cos, worst)
    assert got_tokens == want_tokens, (got_tokens, want_tokens)


@torch.inference_mode()
def test_calibration_hook_equals_one_prefill_per_grid_point():
    """The calibration tool's hook (one sweep per layer: triattention_b200/calibrate.py) on the toy model gives, per layer,
    head and grid point, the error the reference tool's loop computes with one prefill per grid point
    (calibrate.py:46-63 of the reference), and leaves the model's exact output in place."""
    from triattention_b200.calibrate import Calibration, grid
    from triattention_b200.kernels.extension import load_extension
    from triattention_b200.kernels.prefill import Prefill
    from triattention_b200.maps import INF, uniform
    from triattention_b200.models import exact_attention, use_attention
    model = tiny_llama()
    module = load_extension()
    configs, rows = grid()[::7] + [(INF, INF)], 100
    ids = torch.randint(0, 1024, (1, 333), generator=torch.Generator().manual_seed(9)).cuda()
    run = Calibration(Prefill(module, uniform(INF, INF)), configs, rows)
    use_attention(model, "triattention_calibration_test", run.attention)
    swept = model(input_ids=ids, use_cache=False, logits_to_keep=1).logits.float()
    module.check_device_error()
    assert sorted(run.errors) == [0, 1, 2] and all(e.shape == (4, len(configs)) for e in run.errors.values())

    loop = {}
    executors = [Prefill(module, uniform(w8, w4)) for w8, w4 in configs]

    def reference_style(mod, query, key, value, scaling):
        heads, t = query.shape[1], query.shape[2]
        last = slice(max(0, t - rows), t)
        ref = exact_attention(query, key, value, scaling)
        w = mod.o_proj.weight.float()
        wh = w.view(w.shape[0], heads, 128).permute(1, 0, 2)
        gram = wh.transpose(1, 2) @ wh
        exact = ref[0, :, last].float()
        energy = float((exact.transpose(0, 1).reshape(-1, heads * 128) @ w.T).square().sum())
        total = loop.setdefault(mod.layer_idx, torch.zeros(heads, len(configs), dtype=torch.float64))
        for i, prefill in enumerate(executors):
            delta = prefill(mod.layer_idx, query, key, value, scaling)[0, :, last].float() - exact
            total[:, i] += torch.einsum("htd,hde,hte->h", delta, gram, delta).double().cpu() / energy
        return ref

    use_attention(model, "triattention_calibration_loop", reference_style)
    looped = model(input_ids=ids, use_cache=False, logits_to_keep=1).logits.float()
    module.check_device_error()
    assert torch.equal(swept, looped)        # both hooks return the exact attention
    for layer in range(3):
        a, b = run.errors[layer], loop[layer]
        assert torch.isfinite(a).all() and (a >= 0).all()
        # same outputs bit for bit except the grid point without any INT8 tile, summed in another order
        assert torch.allclose(a, b, rtol=2e-2, atol=1e-9), (layer, (a - b).abs().max().item())
    record = run.record("llama", 1)
    assert record["format"] == "triattention-calibration-v1" and record["configs"] == configs and record["rows"] == rows
    assert sorted(record["errors"]) == [0, 1, 2] and len(record["errors"][0]) == 4
