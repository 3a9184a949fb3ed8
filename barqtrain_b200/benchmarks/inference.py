"""Generation benchmark with resident / peak / overhead columns, after the reference's method.

The reference judges its paged KV cache with a ``generate()`` benchmark
(``examples/barqtrain_benchmark_comparison_colab.ipynb``, cell 3 ``benchmark_generation``; method
described in ``README.md:345-364``): warm-up runs, ``cuda_memory_snapshot(reset_peak=True)`` before the
measured loop, a peak snapshot after it, and ``generation_overhead_mb`` = peak allocated minus resident
(``python/barqtrain/memory.py:13-46``).  Two profiles: ``throughput_short`` (short prompt, 64 new tokens,
2 warm-up / 5 measured runs, paged KV off below 512 tokens of cache) and ``memory_long`` (long prompt, 256
new tokens, 1 / 3 runs, paged KV always on).  Columns: ``tokens_per_sec``, ``resident_vram_mb``,
``peak_vram_mb``, ``generation_overhead_mb``, ``paged_kv_cache``.

This module follows that method on a seeded random-weight Llama (there is no network for checkpoints or
tokenizers: prompts are seeded token ids of the profiles' lengths) and compares four set-ups:

``hf_dynamic_cache``            stock ``generate()``: the cache grows by ``torch.cat``
``barq_paged_kv_cache``         the drop-in ``BarqPagedKVCache`` injected by ``patch_inference``
``barq_block_table_gathered``   ``BarqBlockTableCache``: pages from a shared pool, one fused
                                append + gather launch per layer
``barq_block_table_from_pages`` the same cache with decode attention reading the pages directly

The block-table rows add ``pages_peak`` / ``bytes_peak`` of the page pool (``PoolStats``).
"""

from __future__ import annotations

import gc
import os
import statistics
import time
from typing import Dict, List, Optional

import torch

from ..memory import cuda_memory_snapshot, generation_overhead_mb

# Token counts of the reference's prompts: the short prompt is one sentence; the long prompt repeats a
# nine-word sentence 160 times (about 11 tokens each with the reference's tokenizer).
PROFILES = [
    {"profile": "throughput_short", "prompt_tokens": 14, "new_tokens": 64, "warmup_runs": 2, "measure_runs": 5,
     "paged_kv_min_cache_len": 512},
    {"profile": "memory_long", "prompt_tokens": 1760, "new_tokens": 256, "warmup_runs": 1, "measure_runs": 3,
     "paged_kv_min_cache_len": 0},
]
SETUPS = ("hf_dynamic_cache", "barq_paged_kv_cache", "barq_block_table_gathered", "barq_block_table_from_pages")


def build_model(device="cuda", dtype=torch.bfloat16, layers: int = 16, seed: int = 0):
    """A Llama of roughly half a billion parameters with seeded random weights: hidden 1024, 8 query and 2 KV
    heads of dimension 128 (the head shape the from-pages attention kernel serves), 32k vocabulary."""
    from transformers import LlamaConfig, LlamaForCausalLM

    torch.manual_seed(seed)
    cfg = LlamaConfig(vocab_size=32000, hidden_size=1024, intermediate_size=2816, num_hidden_layers=layers,
                      num_attention_heads=8, num_key_value_heads=2, head_dim=128, max_position_embeddings=4096,
                      pad_token_id=0, bos_token_id=1, eos_token_id=None)
    return LlamaForCausalLM(cfg).to(device, dtype).eval()


def _clear_memory() -> None:
    gc.collect()
    torch.cuda.empty_cache()
    torch.cuda.reset_peak_memory_stats()
    torch.cuda.synchronize()


def _generate_kwargs(new_tokens: int) -> Dict:
    # greedy, exactly new_tokens tokens (the model has no EOS token)
    return {"max_new_tokens": new_tokens, "min_new_tokens": new_tokens, "do_sample": False}


def benchmark_generation(setup: str, model, input_ids: torch.Tensor, profile: Dict, page_size: int = 16) -> Dict:
    """One row of the table: the reference's ``benchmark_generation`` for one set-up and profile."""
    from ..hf_block_cache import BarqBlockTableCache, use_paged_attention
    from ..patch_models import patch_inference

    if setup not in SETUPS:
        raise ValueError(f"unknown set-up {setup!r}")
    model.config.use_cache = True
    batch, prompt_tokens = input_ids.shape
    os.environ["BARQTRAIN_ENABLE_PAGED_KV"] = "1"
    os.environ["BARQTRAIN_PAGED_KV_MIN_CACHE_LEN"] = str(profile["paged_kv_min_cache_len"])
    os.environ["BARQTRAIN_PAGED_KV_PAGE_SIZE"] = str(page_size)
    model.config._attn_implementation = "sdpa"
    if setup == "barq_paged_kv_cache":
        patch_inference(model)
    elif setup == "barq_block_table_from_pages":
        use_paged_attention(model)
    last_cache: List[Optional[BarqBlockTableCache]] = [None]

    def run(new_tokens: int):
        kwargs = _generate_kwargs(new_tokens)
        if setup == "hf_dynamic_cache":
            # the stock path must not pick up an injected cache even if the model was patched earlier
            os.environ["BARQTRAIN_ENABLE_PAGED_KV"] = "0"
        elif setup.startswith("barq_block_table"):
            if last_cache[0] is not None:              # the previous run's pool goes before this run's is made
                last_cache[0].release_memory()
            cache = BarqBlockTableCache(model.config, max_batch_size=batch, max_cache_len=prompt_tokens + new_tokens,
                                        page_size=page_size, attention_from_pages=setup.endswith("from_pages"))
            kwargs.update(past_key_values=cache, use_cache=True)
            last_cache[0] = cache
        return model.generate(input_ids, **kwargs)

    _clear_memory()
    with torch.inference_mode():
        for _ in range(profile["warmup_runs"]):
            run(min(16, profile["new_tokens"]))
    if last_cache[0] is not None:
        last_cache[0].release_memory()
    last_cache[0] = None
    _clear_memory()
    resident = cuda_memory_snapshot(reset_peak=True)
    model._barqtrain_last_generate_used_paged_kv = False

    latencies = []
    with torch.inference_mode():
        for _ in range(profile["measure_runs"]):
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            outputs = run(profile["new_tokens"])
            torch.cuda.synchronize()
            latencies.append(time.perf_counter() - t0)
    peak = cuda_memory_snapshot()
    generated = int(outputs.shape[-1] - prompt_tokens)
    avg = sum(latencies) / len(latencies)
    paged = bool(getattr(model, "_barqtrain_last_generate_used_paged_kv", False)) or setup.startswith("barq_block_table")
    row = {
        "profile": profile["profile"], "setup": setup, "dtype": str(model.dtype).replace("torch.", ""),
        "batch": batch, "prompt_tokens": prompt_tokens, "generated_tokens": generated,
        "avg_latency_s": round(avg, 4), "median_latency_s": round(statistics.median(latencies), 4),
        "tokens_per_sec": round(batch * generated / avg, 1) if avg > 0 else 0.0,
        "resident_vram_mb": round(resident.allocated_mb, 1), "peak_vram_mb": round(peak.max_allocated_mb, 1),
        "generation_overhead_mb": round(generation_overhead_mb(resident, peak), 1),
        "paged_kv_cache": paged,
    }
    cache = last_cache[0]
    if cache is not None and cache.store is not None:
        stats = cache.store.stats()
        row["pages_peak"], row["bytes_peak"] = stats.pages_peak, stats.bytes_peak
    model.config._attn_implementation = "sdpa"
    os.environ["BARQTRAIN_ENABLE_PAGED_KV"] = "1"
    return row


def run_table(device="cuda", batch: int = 1, layers: int = 16, profiles=None, setups=SETUPS, page_size: int = 16,
              seed: int = 11) -> List[Dict]:
    """Every set-up on every profile; a fresh model per row, as the reference's ``run_case`` does."""
    rows = []
    g = torch.Generator().manual_seed(seed)
    for profile in profiles or PROFILES:
        ids = torch.randint(2, 32000, (batch, profile["prompt_tokens"]), generator=g).to(device)
        for setup in setups:
            _clear_memory()
            model = build_model(device=device, layers=layers)
            try:
                rows.append(benchmark_generation(setup, model, ids, profile, page_size=page_size))
            finally:
                del model
                _clear_memory()
    return rows


__all__ = ["PROFILES", "SETUPS", "build_model", "benchmark_generation", "run_table"]
