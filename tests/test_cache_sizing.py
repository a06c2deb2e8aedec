"""The size of the cache when no page count is given: arithmetic on an injected figure of free memory
(no GPU), and once on the GPU through the entry point."""
import pytest
import torch

import helpers as H
from vllm_lite_b200.cache import CacheLayout, FixedState, PagedKV
from vllm_lite_b200.cache.sizing import activation_reserve, page_bytes, pages_from_memory, state_bytes
from vllm_lite_b200.config import plan_from_config_json

GiB = 1 << 30


def qwen3_8b_layout():
    need = PagedKV(8, 128)
    return CacheLayout.from_needs([need] * 36, [None] * 36)


def test_a_page_costs_keys_and_values_of_every_layer_of_its_group():
    layout = qwen3_8b_layout()
    assert page_bytes(layout, 16, 2) == [36 * 2 * 8 * 128 * 2 * 16]            # 147,456 bytes a token
    mixed = CacheLayout.from_needs([PagedKV(2, 32), PagedKV(2, 32, window=20), PagedKV(2, 32), FixedState((96,))],
                                   [None] * 4)
    assert page_bytes(mixed, 8, 4) == [2 * 2 * 2 * 32 * 4 * 8, 1 * 2 * 2 * 32 * 4 * 8]
    assert state_bytes(mixed, 10) == 96 * 4 * 10


def test_pages_fill_the_fraction_less_the_reserve():
    layout = qwen3_8b_layout()
    cost = page_bytes(layout, 16, 2)[0]
    pages = pages_from_memory(layout, 16, 2, free_bytes=160 * GiB, fraction=0.9, reserve_bytes=4 * GiB,
                              max_requests=256, max_context=40960)
    assert pages == [(int(160 * GiB * 0.9) - 4 * GiB) // cost]
    assert pages[0] * 16 > 1_000_000                                           # a million tokens of cache, not 16,384
    # a tighter fraction gives fewer pages; an explicit reserve comes off first
    fewer = pages_from_memory(layout, 16, 2, 160 * GiB, 0.5, 4 * GiB, 256, 40960)
    assert fewer[0] < pages[0] and fewer == [(80 * GiB - 4 * GiB) // cost]
    with pytest.raises(ValueError, match="one request"):
        pages_from_memory(layout, 16, 2, 6 * GiB, 0.9, 4 * GiB, 256, 40960)   # 1.4 GiB: not one request of 40,960
    with pytest.raises(ValueError, match="fraction"):
        pages_from_memory(layout, 16, 2, 6 * GiB, 1.5, 0, 256, 40960)


def test_a_group_never_gets_more_pages_than_its_requests_can_hold_and_the_rest_goes_to_the_others():
    layout = CacheLayout.from_needs([PagedKV(2, 32), PagedKV(2, 32, window=20), PagedKV(2, 32)], [None] * 3)
    full, windowed = page_bytes(layout, 8, 2)
    pages = pages_from_memory(layout, 8, 2, free_bytes=64 << 20, fraction=1.0, reserve_bytes=0, max_requests=4,
                              max_context=512, max_step_tokens=64)
    cap = 4 * (-(-(20 + 64) // 8) + 1) + 1
    assert pages[1] == cap                                                     # the window's group is capped ...
    assert pages[0] == min(((64 << 20) - cap * windowed) // full, 4 * 64 + 1)   # ... the other takes what is left
    tight = pages_from_memory(layout, 8, 2, free_bytes=40 * (full + windowed) + 5, fraction=1.0, reserve_bytes=0,
                              max_requests=4, max_context=256, max_step_tokens=64)
    assert tight == [40, 40]                                                   # too little for any cap: even shares


def test_the_reserve_grows_with_the_step_and_with_the_graphs_logits():
    _, plan = plan_from_config_json(dict(H.TINY_B, hidden_size=4096, intermediate_size=12288, num_attention_heads=32,
                                         num_key_value_heads=8, head_dim=128, vocab_size=151936,
                                         max_position_embeddings=40960))
    small = activation_reserve(plan, 512, 8, 4096, 2)
    big = activation_reserve(plan, 4096, 256, 40960, 2)
    assert small < big < 8 * GiB
    assert big - small > 3584 * (4 * 4096 + 2 * (3 * 12288 + 6 * 4096 + 2 * 1024))


@pytest.mark.gpu
def test_the_entry_point_sizes_its_cache_from_the_gpu():
    from vllm_lite_b200 import LLMEngine
    eng = LLMEngine(str(H.model_dir("B")), dtype="bfloat16", block_size=8, max_batch_size=4, max_model_len=256,
                    gpu_memory_fraction=0.02, max_num_batched_tokens=128)
    sized = eng.runner.sized_from_memory
    assert sized is not None and sized["fraction"] == 0.02
    budget = int(sized["free_bytes"] * 0.02) - sized["reserve_bytes"]
    assert budget > 0, "2 % of a free B200 exceeds the tiny model's reserve"
    # capped by what 4 requests of 256 tokens could hold, which is far below 2 % of the GPU
    assert sized["pages"] == [4 * 32 + 1]
    assert eng.runner.storage.bytes() <= budget
    out = eng.generate([H.tokens_for("B", 20, 1)], max_tokens=5)
    assert len(out[0]) == 5
    explicit = LLMEngine(str(H.model_dir("B")), dtype="bfloat16", block_size=8, kv_blocks=48, max_batch_size=4)
    assert explicit.runner.sized_from_memory is None and explicit.runner.cache.free_pages() == [48]
