"""Prefix cache of the rollout engine: prompts that start with pages another request left behind (same prompt again, the
next turn of a conversation) are prefilled from the first uncached token and produce the same tokens and log-probs."""
import torch

from verl_b200.models import get_preset
from verl_b200.models.weights import FlatParams
from verl_b200.workers.rollout.native.engine import RolloutEngine, SamplingParams


def _params(name="tiny-qwen2", seed=3):
    cfg = get_preset(name)
    P = FlatParams(cfg, dtype=torch.float32)
    P.init_weights(seed=seed, std=0.1)
    return cfg, P


def _engine(cfg, P, cache, **kw):
    kw.setdefault("num_blocks", 64)
    return RolloutEngine(cfg, P, max_num_seqs=4, max_model_len=96, block_size=8, sync_interval=2, eos_token_id=-1,
                         enable_prefix_caching=cache, **kw)


def _same(a, b, atol=1e-4):
    assert [o.token_ids for o in a] == [o.token_ids for o in b]
    for x, y in zip(a, b):
        assert torch.allclose(torch.tensor(x.log_probs), torch.tensor(y.log_probs), atol=atol)


def test_repeated_prompt_and_next_turn_hit_the_cache():
    cfg, P = _params()
    plain, cached = _engine(cfg, P, False), _engine(cfg, P, True)
    g = torch.Generator().manual_seed(0)
    p1 = torch.randint(3, 500, (29,), generator=g).tolist()
    sp = SamplingParams(temperature=0.0, max_tokens=12)
    a1, b1 = plain.generate([p1], sp), cached.generate([p1], sp)
    _same(a1, b1)
    assert cached.stats.get("prefix_cache_hit_tokens", 0) == 0
    # the same prompt again: its three full pages are cached, five tokens are computed (the last one always is)
    before = cached.stats["prefill_tokens"]
    _same(plain.generate([p1], sp), cached.generate([p1], sp))
    assert cached.stats["prefix_cache_hit_tokens"] == 24 and cached.stats["prefill_tokens"] - before == 5
    # next turn: prompt + response + a tool reply; the pages the response filled are cached as well
    p2 = p1 + a1[0].token_ids + torch.randint(3, 500, (7,), generator=g).tolist()
    hits = cached.stats["prefix_cache_hit_tokens"]
    _same(plain.generate([p2], sp), cached.generate([p2], sp))
    assert cached.stats["prefix_cache_hit_tokens"] - hits == (29 + 12 - 1) // 8 * 8
    # a prompt that diverges inside the second page reuses only the first
    p3 = p1[:12] + [7, 7, 7] + p1[15:]
    hits = cached.stats["prefix_cache_hit_tokens"]
    _same(plain.generate([p3], sp), cached.generate([p3], sp))
    assert cached.stats["prefix_cache_hit_tokens"] - hits == 8


def test_groups_sampling_and_mixed_batches():
    cfg, P = _params()
    plain, cached = _engine(cfg, P, False), _engine(cfg, P, True)
    g = torch.Generator().manual_seed(1)
    sysp = torch.randint(3, 500, (20,), generator=g).tolist()                  # a shared system prompt
    prompts = [sysp + torch.randint(3, 500, (n,), generator=g).tolist() for n in (5, 9, 3)]
    sp = SamplingParams(temperature=1.0, top_k=50, max_tokens=10, seed=5)
    cached.generate([prompts[0]], sp)                                          # warms the cache with the system prompt's pages
    batch = [prompts[1], prompts[1], prompts[2], prompts[0]]                   # a group of two, a new tail, an exact repeat
    sps = [SamplingParams(temperature=1.0, top_k=50, max_tokens=10, seed=s) for s in (5, 6, 7, 8)]
    _same(plain.generate(batch, sps), cached.generate(batch, sps))
    assert cached.stats["prefix_cache_hit_tokens"] >= 16 * 3 and not cached.running
    # every page is accounted for: free, or idle in the cache
    assert len(cached.free_blocks) + len(cached._idle_cached) == cached.num_blocks and not cached._block_users


def test_eviction_and_weight_updates():
    cfg, P = _params()
    plain, cached = _engine(cfg, P, False, num_blocks=12), _engine(cfg, P, True, num_blocks=12)
    g = torch.Generator().manual_seed(2)
    sp = SamplingParams(temperature=0.0, max_tokens=8)
    prompts = [torch.randint(3, 500, (25,), generator=g).tolist() for _ in range(6)]
    for p in prompts + prompts[:2]:                                            # more distinct pages than the pool holds
        _same(plain.generate([p], sp), cached.generate([p], sp))
    assert len(cached._page_of_hash) == len(cached._hash_of_page) <= 12
    assert len(cached.free_blocks) + len(cached._idle_cached) == 12
    # new weights: cached content is stale and must not be used
    P.flat.mul_(1.05)
    plain.clear_kv_cache()
    cached.clear_kv_cache()
    assert not cached._page_of_hash and not cached._idle_cached
    hits = cached.stats.get("prefix_cache_hit_tokens", 0)
    _same(plain.generate([prompts[1]], sp), cached.generate([prompts[1]], sp))
    assert cached.stats.get("prefix_cache_hit_tokens", 0) == hits
