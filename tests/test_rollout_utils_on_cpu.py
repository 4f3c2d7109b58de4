import asyncio
from types import SimpleNamespace

import pytest

from verl_b200.workers.rollout.utils import (dedup_vision_placeholder_runs, ensure_async_iterator, get_max_position_embeddings,
                                             get_vision_placeholder_token_ids, qwen2_5_vl_dedup_image_tokens)


def test_context_length_of_text_and_vision_language_configs():
    assert get_max_position_embeddings(SimpleNamespace(max_position_embeddings=4096)) == 4096
    assert get_max_position_embeddings(SimpleNamespace(text_config=SimpleNamespace(max_position_embeddings=32768))) == 32768
    with pytest.raises(ValueError):
        get_max_position_embeddings(SimpleNamespace())


def test_async_iteration_over_both_kinds_of_iterables():
    async def agen():
        for i in range(3):
            yield i

    async def collect(it):
        return [x async for x in ensure_async_iterator(it)]

    assert asyncio.run(collect([1, 2])) == [1, 2] and asyncio.run(collect(agen())) == [0, 1, 2]


def test_placeholder_ids_and_run_collapse():
    class Qwen2VLImageProcessorFast:
        pass

    proc = SimpleNamespace(image_processor=Qwen2VLImageProcessorFast(), image_token_id=7, video_token_id=8)
    assert get_vision_placeholder_token_ids(proc) == [7, 8] and get_vision_placeholder_token_ids(None) == []
    ids = [1, 5, 7, 7, 7, 6, 2, 5, 8, 8, 6, 7, 3]
    assert qwen2_5_vl_dedup_image_tokens(ids, proc) == [1, 5, 7, 6, 2, 5, 8, 6, 7, 3]
    assert qwen2_5_vl_dedup_image_tokens(ids, SimpleNamespace(image_processor=object(), image_token_id=7)) == ids
    assert dedup_vision_placeholder_runs([], [7]) == [] and dedup_vision_placeholder_runs([7, 7], []) == [7, 7]
    # ids looked up through the tokenizer when the processor only names the token
    tok = SimpleNamespace(convert_tokens_to_ids=lambda t: {"<img>": 11}[t])
    assert get_vision_placeholder_token_ids(SimpleNamespace(image_token="<img>", tokenizer=tok)) == [11]
