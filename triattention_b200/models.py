"""Model glue: Hugging Face attention hook, ``TriAttention`` and the greedy generate loop.

Mirrors ``triattention/models.py`` (same function names and signatures).  Additions: ``generate``
accepts a batch of equal-length prompts and keeps the argmax on the device; with a batch of one it
returns a flat token list like the reference (``models.py:72-85``), otherwise one list per sequence.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F
import transformers
from torch.nn.attention import SDPBackend, sdpa_kernel
from transformers import AutoConfig, AutoTokenizer
from transformers.modeling_utils import ALL_ATTENTION_FUNCTIONS

from triattention_b200.kernels.decode import DecodeCache
from triattention_b200.kernels.extension import LONG_TAIL_ROWS, load_extension
from triattention_b200.kernels.prefill import Prefill
from triattention_b200.maps import load_map, preset


def load_tokenizer(path):
    mistral = AutoConfig.from_pretrained(path).model_type == "mistral3"
    return AutoTokenizer.from_pretrained(path, **({"fix_mistral_regex": True} if mistral else {}))


def load_model(path):
    """models.py:20-32, including the YaRN x4 patch for qwen2."""
    config = AutoConfig.from_pretrained(path)
    if config.model_type == "qwen2":
        theta = config.rope_parameters["rope_theta"]
        config.rope_parameters = dict(rope_type="yarn", factor=4.0, original_max_position_embeddings=32768,
                                      rope_theta=theta)
        config.max_position_embeddings = 4 * 32768
    loader = transformers.AutoModelForImageTextToText if hasattr(config, "vision_config") else transformers.AutoModelForCausalLM
    return loader.from_pretrained(path, config=config, dtype=torch.bfloat16).cuda().eval()


def render_prompt(tokenizer, prompt):
    return tokenizer.apply_chat_template([{"role": "user", "content": prompt}], tokenize=False,
                                         add_generation_prompt=True, date_string="30 Jul 2026")


def eos_ids(tokenizer, model):
    as_set = lambda ids: set(ids if isinstance(ids, list) else [ids])
    return as_set(tokenizer.eos_token_id) | as_set(model.generation_config.eos_token_id)


def exact_attention(query, key, value, scaling):
    with sdpa_kernel([SDPBackend.FLASH_ATTENTION]):
        return F.scaled_dot_product_attention(query, key, value, is_causal=True, scale=scaling, enable_gqa=True)


def use_attention(model, name, fn):
    def attention(module, query, key, value, attention_mask, scaling, dropout=0.0, **kwargs):
        return fn(module, query, key, value, scaling).transpose(1, 2).contiguous(), None

    ALL_ATTENTION_FUNCTIONS[name] = attention
    model.set_attn_implementation(name)


class TriAttention:
    def __init__(self, model, qk_map=None, max_new_tokens=256, fold_tail=False):
        """fold_tail=False is the reference: generated tokens stay in a BF16 tail, so max_new_tokens <= 1024
        (models.py:58-70, common_host.cuh:56).  fold_tail=True lifts the cap: every 64 generated tokens are quantised
        into one more cached tile (DecodeCache(fold_tail=...)); numerics then differ from the reference's."""
        self.model = model
        module = load_extension()
        self.module = module
        self.decode_cache = (DecodeCache(module, max_tail=64, fold_tail=max_new_tokens) if fold_tail
                             else DecodeCache(module, max_tail=max_new_tokens))
        bands_fn = qk_map if callable(qk_map) else load_map(qk_map or preset(model), model)
        self.prefill = Prefill(module, bands_fn, self.decode_cache)

        def attention(mod, query, key, value, scaling):
            if query.shape[2] == 1 and self.decode_cache.stored(mod.layer_idx):
                return self.decode_cache(mod.layer_idx, query, key, value, scaling)
            return self.prefill(mod.layer_idx, query, key, value, scaling)

        use_attention(model, "triattention", attention)

    @torch.inference_mode()
    def generate(self, ids, max_new_tokens, eos=(), cuda_graph=False):
        """Greedy decoding (models.py:72-85 of the reference, batched).  cuda_graph=True captures one decode step of
        the whole model (every layer's projections, the two decode launches per layer, argmax, position and step
        counters) in a CUDA graph and replays it per token: the reference launches layer by layer from Python and
        synchronises with the host for every token."""
        batch, device = ids.shape[0], ids.device
        out = self.model(input_ids=ids, use_cache=False, logits_to_keep=1)
        eos_t = torch.tensor(sorted(eos), dtype=torch.long, device=device)
        alive = torch.ones(batch, dtype=torch.bool, device=device)
        history = []
        token = out.logits[:, -1].argmax(-1)
        replay = None
        if cuda_graph and self.decode_cache.reserve:
            raise RuntimeError("cuda_graph replays fixed cache tables; it cannot be combined with fold_tail")
        if cuda_graph and max_new_tokens > 1:
            tok = token[:, None].clone()
            pos = torch.full((batch, 1), ids.shape[1], device=device)

            def step():
                logits = self.model(input_ids=tok, position_ids=pos, use_cache=False).logits
                tok.copy_(logits[:, -1].argmax(-1)[:, None])
                pos.add_(1)
                self.decode_cache.advance()

            # A graph replays the merge kernel chosen at capture, whatever the tail has grown to: the one for short tails
            # only where the whole generation is short.
            # One eager run on a side stream first (library workspaces, lazy initialisation, the kernels loaded).  It
            # appends this token's K / V to the tails at the current step index, which the captured step then simply
            # writes again; the counters it moved are put back.
            self.decode_cache.hint_rows = 1 if max_new_tokens <= 2 * LONG_TAIL_ROWS else -1
            try:
                side = torch.cuda.Stream(device)
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    step()
                    tok.copy_(token[:, None])
                    pos.sub_(1)
                    self.decode_cache.step.sub_(1)
                torch.cuda.current_stream().wait_stream(side)
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    step()
            finally:
                self.decode_cache.hint_rows = None
            replay = graph.replay
        for i in range(max_new_tokens):
            if eos_t.numel():
                alive &= ~torch.isin(token, eos_t)
                if batch == 1 and not bool(alive[0]):
                    break
            history.append(torch.where(alive, token, torch.full_like(token, -1)))
            if i + 1 == max_new_tokens:
                break
            if replay is not None:
                replay()
                token = tok[:, 0].clone()
            else:
                position = torch.full((batch, 1), ids.shape[1] + i, device=device)
                out = self.model(input_ids=token[:, None], position_ids=position, use_cache=False)
                self.decode_cache.advance()
                token = out.logits[:, -1].argmax(-1)
        self.module.check_device_error(device)
        if not history:
            return [] if batch == 1 else [[] for _ in range(batch)]
        tokens = torch.stack(history, 1).cpu()
        rows = []
        for row in tokens.tolist():
            rows.append(row[:row.index(-1)] if -1 in row else row)
        return rows[0] if batch == 1 else rows
