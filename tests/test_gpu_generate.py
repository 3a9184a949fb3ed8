"""The paged cache under Hugging Face ``generate()`` on a tiny random Llama: the tokens and the final
logits must match the stock dynamic cache (the cache copies K/V bit for bit, so attention sees the
same values; the operands differ only in stride)."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _tiny_llama():
    from transformers import LlamaConfig, LlamaForCausalLM

    torch.manual_seed(0)
    cfg = LlamaConfig(vocab_size=211, hidden_size=128, intermediate_size=256, num_hidden_layers=3,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=32, max_position_embeddings=512,
                      pad_token_id=0, bos_token_id=1, eos_token_id=None)
    return LlamaForCausalLM(cfg).to("cuda").eval()


def test_generate_with_paged_cache_matches_dynamic_cache(monkeypatch):
    from barqtrain_b200 import BarqPagedKVCache, _ffi, create_paged_kv_cache
    from barqtrain_b200.patch_models import patch_inference

    backend = _ffi.require_cuda_backend()
    model = _tiny_llama()
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(2, 211, (2, 37), generator=g).to("cuda")
    new_tokens = 24
    with torch.no_grad():
        want = model.generate(ids, max_new_tokens=new_tokens, do_sample=False)

        launches = backend.launches
        cache = create_paged_kv_cache(model, max_batch_size=2, max_cache_len=37 + new_tokens, page_size=16)
        got = model.generate(ids, max_new_tokens=new_tokens, do_sample=False, past_key_values=cache, use_cache=True)
    assert torch.equal(got, want)
    # one native append per layer per forward: prompt pass + one pass per further token fed back
    assert backend.launches - launches == 3 * new_tokens
    assert cache.get_seq_length() == 37 + new_tokens - 1
    assert cache.layers[0].seq_lens.cpu().tolist() == [37 + new_tokens - 1] * 2

    # the reference's injection route: patch once, then plain generate() picks the paged cache up
    monkeypatch.setenv("BARQTRAIN_PAGED_KV_MIN_CACHE_LEN", "0")
    patch_inference(model)
    assert model._barqtrain_paged_kv_supported and model._barqtrain_generate_paged_kv_patched
    with torch.no_grad():
        again = model.generate(ids, max_new_tokens=new_tokens, do_sample=False)
    assert model._barqtrain_last_generate_used_paged_kv is True
    assert torch.equal(again, want)
    monkeypatch.setenv("BARQTRAIN_PAGED_KV_MIN_CACHE_LEN", "256")
    with torch.no_grad():
        short = model.generate(ids, max_new_tokens=4, do_sample=False)
    assert model._barqtrain_last_generate_used_paged_kv is False and short.shape == (2, 41)
    assert isinstance(cache, BarqPagedKVCache) and backend.read_status("cuda") == 0


def _llama_128():
    from transformers import LlamaConfig, LlamaForCausalLM

    torch.manual_seed(1)
    cfg = LlamaConfig(vocab_size=199, hidden_size=512, intermediate_size=512, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=128, max_position_embeddings=512,
                      pad_token_id=0, bos_token_id=1, eos_token_id=None)
    return LlamaForCausalLM(cfg).to("cuda", torch.bfloat16).eval()


@pytest.mark.parametrize("from_pages", [False, True])
def test_block_table_cache_under_generate(from_pages):
    """The block-table cache as a ``transformers`` cache: prefill + decode logits must match the stock
    dynamic cache - exactly when attention runs on the gathered tensors (same values, same SDPA call),
    within bf16 attention tolerance when decode attention reads the pages directly."""
    from transformers import DynamicCache

    from barqtrain_b200 import _ffi
    from barqtrain_b200.hf_block_cache import BarqBlockTableCache, use_paged_attention

    backend = _ffi.require_cuda_backend()
    model = _llama_128()
    g = torch.Generator().manual_seed(9)
    ids = torch.randint(2, 199, (3, 45), generator=g).to("cuda")
    steps = 20

    def run(cache):
        logits = []
        with torch.no_grad():
            out = model(ids, past_key_values=cache, use_cache=True)
            logits.append(out.logits[:, -1].float())
            tok = out.logits[:, -1].argmax(-1, keepdim=True)
            fed = [tok]
            for _ in range(steps):
                out = model(fed[-1], past_key_values=cache, use_cache=True)
                logits.append(out.logits[:, -1].float())
                fed.append(forced[len(fed)] if forced is not None else out.logits[:, -1].argmax(-1, keepdim=True))
        return logits, fed

    forced = None
    want, fed = run(DynamicCache(config=model.config))
    forced = fed                                        # feed the same tokens so the runs stay comparable
    if from_pages:
        use_paged_attention(model)
    launches = backend.launches
    cache = BarqBlockTableCache(model.config, max_batch_size=3, max_cache_len=45 + steps + 1, page_size=16,
                                attention_from_pages=from_pages)
    got, _ = run(cache)
    assert backend.launches > launches
    assert cache.get_seq_length() == 45 + steps
    assert cache.store.stats().pages_resident == 3 * -(-(45 + steps) // 16)
    for i, (a, b) in enumerate(zip(got, want)):
        if from_pages:
            assert torch.allclose(a, b, atol=6e-2, rtol=5e-2), (i, (a - b).abs().max().item())
        else:
            assert torch.equal(a, b), (i, (a - b).abs().max().item())
    # generate() end to end runs on it as well
    with torch.no_grad():
        out = model.generate(ids, max_new_tokens=8, do_sample=False,
                             past_key_values=BarqBlockTableCache(model.config, 3, 45 + 8, 16, from_pages), use_cache=True)
    assert out.shape == (3, 53)
    model.config._attn_implementation = "sdpa"
    assert backend.read_status("cuda") == 0


def test_generation_benchmark_table_has_the_reference_columns_and_paged_rows():
    """``benchmarks.inference`` follows the reference's ``benchmark_generation`` (notebook cell 3): every row
    carries the reference's columns; the paged set-ups report ``paged_kv_cache`` on the long profile; and the
    block-table cache read from the pages adds no more generation overhead than the stock dynamic cache."""
    from barqtrain_b200 import _ffi
    from barqtrain_b200.benchmarks import inference

    backend = _ffi.require_cuda_backend()
    profile = {"profile": "memory_long", "prompt_tokens": 700, "new_tokens": 40, "warmup_runs": 1, "measure_runs": 1,
               "paged_kv_min_cache_len": 0}
    rows = inference.run_table(device="cuda", batch=2, layers=2, profiles=[profile])
    by = {r["setup"]: r for r in rows}
    assert set(by) == set(inference.SETUPS)
    for r in rows:
        for column in ("tokens_per_sec", "resident_vram_mb", "peak_vram_mb", "generation_overhead_mb", "paged_kv_cache"):
            assert column in r
        assert r["generated_tokens"] == 40 and r["tokens_per_sec"] > 0
        assert r["peak_vram_mb"] >= r["resident_vram_mb"] > 0
    assert by["hf_dynamic_cache"]["paged_kv_cache"] is False
    assert all(by[s]["paged_kv_cache"] is True for s in inference.SETUPS[1:])
    assert by["barq_block_table_from_pages"]["pages_peak"] == 2 * -(-740 // 16)
    # the page pool is sized for the whole generation, like the stock cache's final tensors: the two overheads are
    # of one size (the stock cache adds torch.cat transients, the pool its table and a partly used last page)
    assert by["barq_block_table_from_pages"]["generation_overhead_mb"] <= 1.15 * by["hf_dynamic_cache"]["generation_overhead_mb"] + 2
    # short profile: the injection stays off below its minimum cache length, as in the reference
    short = dict(inference.PROFILES[0], warmup_runs=1, measure_runs=1, new_tokens=8)
    row = inference.benchmark_generation("barq_paged_kv_cache", inference.build_model(layers=2), torch.randint(
        2, 32000, (1, 14)).to("cuda"), short)
    assert row["paged_kv_cache"] is False
    assert backend.read_status("cuda") == 0
