"""In-process rollout engine: continuous batching over a paged KV cache with a device-resident decode loop.

Design (one engine per GPU, or per tensor-parallel group):

* **Shared weights.** The engine reads the trainer's bf16 working parameters in place (``FlatParams``);
  a weight update is visible to the next generation call without any copy or re-layout.
* **Slots.** ``max_num_seqs`` sequence slots with static per-slot state tensors on the device (current
  token, position, context length, generated count, active flag, block-table row).  A decode step runs
  over *all* slots with static shapes, so the whole step (28 layers + LM head + sampler + state update)
  is one CUDA graph; inactive slots cost nothing in attention (context length 0) and their GEMM rows
  are ignored.
* **Device-resident loop.** Sampled tokens feed the next step on the device; EOS / length termination
  is evaluated on the device.  The host synchronises only every ``sync_interval`` steps to retire
  finished sequences and admit waiting ones (continuous batching at that granularity).
* **Paged KV.** Blocks of ``block_size`` tokens from one pool ``[layers, 2, blocks, block_size, kv_heads,
  head_dim]``; a sequence reserves the blocks for ``prompt + max_new_tokens`` at admission and returns
  them when it retires.  ``release_kv_cache`` / ``resume_kv_cache`` hand the pool's memory back to the
  trainer between rollout phases.
* **Prefill** runs the packed varlen forward of the training model with a hook that scatters rotated
  K/V into the cache, in chunks of at most ``max_num_batched_tokens`` tokens.

Feature parity target: how the reference drives vLLM (``verl/workers/rollout/vllm_rollout/
vllm_async_server.py:254-720``: token-in/token-out generate, sampling params, log-probs of sampled tokens,
max_num_seqs / max_num_batched_tokens, dummy-weight start, KV release/resume, abort).
"""

from __future__ import annotations

import math
import os
import time
import zlib
from collections import OrderedDict, deque
from dataclasses import dataclass, field
from typing import Optional, Sequence

import torch
import torch.distributed as dist

from ....models.config import ModelConfig
from ....models.decoder import DecoderModel, PackedBatch, TensorParallelShard
from ....models.weights import FlatParams
from ....ops import functional as F

__all__ = ["SamplingParams", "RequestOutput", "RolloutEngine"]


@dataclass
class SamplingParams:
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = -1
    max_tokens: int = 128
    ignore_eos: bool = False
    stop_token_ids: Sequence[int] = ()
    logprobs: bool = True
    seed: Optional[int] = None
    repetition_penalty: float = 1.0


@dataclass
class RequestOutput:
    request_id: str
    prompt_ids: list[int]
    token_ids: list[int]
    log_probs: Optional[list[float]]
    stop_reason: str  # completed | length | aborted
    num_preempted: int = 0
    extra_fields: dict = field(default_factory=dict)


@dataclass
class _Request:
    rid: str
    prompt: list[int]
    params: SamplingParams
    slot: int = -1
    blocks: list[int] = field(default_factory=list)
    arrival: float = 0.0
    handoff: Optional[dict] = None  # prefilled elsewhere: KV content, first token and sampler state arrive with the request
    cached: int = 0                 # leading prompt tokens whose pages came from the prefix cache


class RolloutEngine:
    def __init__(self, cfg: ModelConfig, params: FlatParams, *, max_num_seqs: int = 256,
                 max_num_batched_tokens: int = 8192, max_model_len: int = 4096, block_size: int = 64,
                 num_blocks: Optional[int] = None, gpu_memory_utilization: float = 0.5, eos_token_id=None,
                 valid_vocab_size: int = 0, use_cuda_graph: bool = True, sync_interval: int = 16, seed: int = 0,
                 tp_group=None, quantization: Optional[str] = None, share_prefill: bool = True, record_routing: bool = False,
                 enable_prefix_caching: bool = False):
        """``tp_group``: process group of the ranks that serve the same requests tensor-parallel (each holds the
        full replicated weights and uses its shard of them in place; see ``TensorParallelShard``). All ranks of the
        group must be fed the same requests in the same order."""
        self.cfg = cfg
        assert quantization in (None, "", "fp8"), f"unsupported rollout quantization: {quantization}"
        self.quantization = quantization or None
        self.share_prefill = bool(share_prefill)
        # Prefix cache across requests: full pages stay indexed by a chain hash of their tokens after their last user has
        # finished (evicted least-recently-used when fresh pages run out); a new prompt that starts with cached pages (the
        # next turn of a conversation, a shared system prompt) points at them and is prefilled from the first uncached token.
        # Emptied with every weight update. Off with routing recording (a cached page has no routing record).
        self.enable_prefix_caching = bool(enable_prefix_caching) and not (bool(record_routing) and cfg.is_moe)
        self._page_of_hash: dict = {}      # chain hash -> page
        self._hash_of_page: dict = {}      # page -> chain hash
        self._idle_cached: "OrderedDict[int, None]" = OrderedDict()   # indexed pages without a user, oldest first
        # mixture-of-experts models: return the experts every router picked for every token that went through the model
        # (``RequestOutput.extra_fields["routed_experts"]``, [prompt + generated - 1, layers, k]) for router replay
        self.record_routing = bool(record_routing) and cfg.is_moe
        self.out_routed = None
        self.tp_group = tp_group
        self.tp_size = dist.get_world_size(tp_group) if tp_group is not None else 1
        self.tp_rank = dist.get_rank(tp_group) if tp_group is not None else 0
        assert cfg.num_key_value_heads % self.tp_size == 0 and (cfg.is_moe or cfg.intermediate_size % (8 * self.tp_size) == 0), \
            "tensor-parallel size must divide the KV heads and the MLP width"
        self.params = params
        self.device = params.flat.device
        self.is_cuda = self.device.type == "cuda"
        self.S = int(max_num_seqs)
        self.max_batched = int(max_num_batched_tokens)
        self.max_model_len = int(max_model_len)
        self.bs = int(block_size)
        self.max_blocks_per_seq = (self.max_model_len + self.bs - 1) // self.bs
        self.eos = eos_token_id if eos_token_id is not None else cfg.eos_token_id
        self.valid_vocab = valid_vocab_size or cfg.vocab_size
        self.use_graph = bool(use_cuda_graph) and self.is_cuda
        self.sync_interval = max(1, int(sync_interval))
        self.gpu_memory_utilization = gpu_memory_utilization
        self._num_blocks_req = num_blocks
        self.model = DecoderModel(cfg, params, max_positions=self.max_model_len + 1)
        self.model.kv_hook = self._prefill_kv_hook
        self._tp_share = None
        if self.tp_size > 1:
            assert not cfg.is_moe, "tensor-parallel rollout of MoE models is not implemented (use expert parallelism)"
            self.model.tp = TensorParallelShard(self.tp_rank, self.tp_size, self._make_row_linear())
        self.kv: Optional[torch.Tensor] = None
        self.free_blocks: list[int] = []
        self._block_users: dict[int, int] = {}  # prompt pages shared by several sequences -> number of users
        self._graph = None
        self._graph_key = None
        self._seed = seed
        self._rid = 0
        self.waiting: deque[_Request] = deque()
        self.running: dict[int, _Request] = {}
        self.finished: list[RequestOutput] = []
        self.stats = dict(prefill_tokens=0, decode_steps=0, generated_tokens=0, prefill_s=0.0, decode_s=0.0)
        self._decode_events: list = []
        self._alloc_state()
        self.resume_kv_cache()
        if self.quantization == "fp8":
            self.model.quantize_linear_weights_fp8()

    def _make_row_linear(self):
        """Row-parallel linear summed over the tensor-parallel group. GPUs: one kernel (GEMM with the all-reduce in its
        epilogue over peer memory). CPU: GEMM followed by a gloo all-reduce (used by the multi-process tests)."""
        if self.is_cuda:
            from ....parallel.symmetric import FusedRowParallelLinear

            fused = FusedRowParallelLinear(max(self.max_batched, self.S), self.cfg.hidden_size, self.device, self.tp_group)
            self._fused_row = fused
            # decode: every rank of the group computes the logits of, and samples, its own share of the sequences; the
            # tokens and log-probs are shared over peer memory (VERL_B200_TP_SPLIT_SAMPLING=0: every rank samples all)
            if self.S % self.tp_size == 0 and os.environ.get("VERL_B200_TP_SPLIT_SAMPLING", "1") != "0":
                from ....parallel.symmetric import PeerShare

                self._tp_share = PeerShare(2 * (self.S // self.tp_size), self.device, self.tp_group)
            return lambda a, w, bias: fused(a, w, bias)

        def row_linear(a, w, bias):
            y = a.float() @ w.float().t()
            dist.all_reduce(y, group=self.tp_group)
            if bias is not None:
                y = y + bias.float()
            return y.to(a.dtype)

        return row_linear

    # ------------------------------------------------------------------------------------ memory
    def kv_bytes_per_block(self) -> int:
        c = self.cfg
        return c.num_hidden_layers * 2 * self.bs * (c.kv_size // self.tp_size) * self.params.flat.element_size()

    def resume_kv_cache(self) -> None:
        if self.kv is not None:
            return
        c = self.cfg
        n = self._num_blocks_req
        if n is None:
            if self.is_cuda:
                torch.cuda.empty_cache()  # cached-but-unused allocator blocks would otherwise count as occupied
                free, total = torch.cuda.mem_get_info(self.device)
                budget = min(free - (2 << 30), int(total * self.gpu_memory_utilization))
                n = max(self.max_blocks_per_seq, int(budget // self.kv_bytes_per_block()))
            else:
                n = self.S * self.max_blocks_per_seq
            n = min(n, self.S * self.max_blocks_per_seq + 1)
        if self.tp_size > 1:  # identical admission decisions on every rank of the group need identical pool sizes
            t = torch.tensor([int(n)], dtype=torch.int64, device=self.device)
            dist.all_reduce(t, op=dist.ReduceOp.MIN, group=self.tp_group)
            n = int(t.item())
        self.num_blocks = int(n)
        self.kv = torch.zeros(c.num_hidden_layers, 2, self.num_blocks, self.bs, c.num_key_value_heads // self.tp_size, c.head_dim,
                              dtype=self.params.flat.dtype, device=self.device)
        self.free_blocks = list(range(self.num_blocks - 1, -1, -1))
        self._block_users = {}
        self._graph = None  # cache addresses changed

    def _release_blocks(self, blocks: list[int]) -> None:
        """Give blocks back; a prompt page shared by the samples of a group is free once its last user is done."""
        shared = self._block_users
        for b in blocks:
            n = shared.get(b)
            if n is not None and n > 1:
                shared[b] = n - 1
                continue
            if n is not None:
                del shared[b]
            if b in self._hash_of_page:
                self._idle_cached[b] = None      # content stays valid: reusable until evicted
            else:
                self.free_blocks.append(b)

    def _take_block(self) -> int:
        """A fresh page: from the free list, else the least recently used idle page of the prefix cache."""
        if self.free_blocks:
            return self.free_blocks.pop()
        b, _ = self._idle_cached.popitem(last=False)
        del self._page_of_hash[self._hash_of_page.pop(b)]
        return b

    def _page_hashes(self, tokens: Sequence[int], n_pages: int) -> list:
        """Chain hash of each of the first ``n_pages`` full pages of ``tokens`` (a page's hash covers everything before it)."""
        import hashlib
        from array import array

        out, h = [], b""
        for i in range(n_pages):
            h = hashlib.blake2b(h + array("q", tokens[i * self.bs : (i + 1) * self.bs]).tobytes(), digest_size=16).digest()
            out.append(h)
        return out

    def _index_pages(self, tokens: Sequence[int], blocks: list[int], n_valid: int) -> None:
        """Index the pages of ``blocks`` that ``tokens[:n_valid]`` fill completely (their content is final)."""
        for i, h in enumerate(self._page_hashes(tokens, min(n_valid // self.bs, len(blocks)))):
            b = blocks[i]
            if h not in self._page_of_hash and b not in self._hash_of_page:
                self._page_of_hash[h] = b
                self._hash_of_page[b] = h

    def _drop_prefix_cache(self) -> None:
        self._page_of_hash.clear()
        self._hash_of_page.clear()
        self._idle_cached.clear()

    def release_kv_cache(self) -> None:
        assert not self.running, "cannot release the KV cache with sequences in flight"
        self.kv = None
        self._graph = None
        self.free_blocks = []
        self._block_users = {}
        self._drop_prefix_cache()
        if self.is_cuda:
            torch.cuda.empty_cache()

    def clear_kv_cache(self) -> None:
        """Forget all cached content (called after every weight update)."""
        assert not self.running
        if self.quantization == "fp8":
            self.model.quantize_linear_weights_fp8()  # the bf16 weights changed: refresh the e4m3 copies
            self._graph = None
        self._drop_prefix_cache()
        if self.kv is not None:
            self.free_blocks = list(range(self.num_blocks - 1, -1, -1))
            self._block_users = {}

    def _alloc_state(self) -> None:
        S, dev = self.S, self.device
        z = lambda dt: torch.zeros(S, dtype=dt, device=dev)
        self.tok, self.pos, self.ctx, self.gen = z(torch.int64), z(torch.int32), z(torch.int32), z(torch.int32)
        self.max_new = z(torch.int32)
        self.active = z(torch.bool)
        self.ignore_eos = z(torch.bool)
        self.seeds = z(torch.int64)
        self.stop_ids = torch.full((S, 8), -1, dtype=torch.int64, device=dev)  # per slot: extra tokens that end the sequence
        self.rep_penalty = torch.ones(S, dtype=torch.float32, device=dev)
        self.seen = None            # [S, vocab] bool, allocated when a request asks for a repetition penalty
        self._use_penalty = False
        self.block_table = torch.zeros(S, self.max_blocks_per_seq, dtype=torch.int32, device=dev)
        self.out_cap = 0
        self.out_tok = self.out_lp = None
        self.temperature = 1.0
        self.top_k, self.top_p = -1, 1.0
        self.free_slots = list(range(S - 1, -1, -1))
        # grouped decode attention: the samples of a prompt share its full pages; a group kernel reads them once per group
        # (``ops.paged_decode_grouped``). Host mirror: group id -> member slots, slot -> group id. Off by default: measured at
        # 320 sequences x 2048 tokens of context in groups of 5, the per-sequence kernel already finds the shared pages in L2
        # (12.5 ms per decode step) and the group kernel, whose warps walk a page's 64 tokens one after the other, does not
        # beat that (12.9 ms); VERL_B200_GROUPED_DECODE=1 turns it on.
        nh_l = self.cfg.num_attention_heads // self.tp_size
        nkv_l = self.cfg.num_key_value_heads // self.tp_size
        # VERL_B200_FUSED_ROPE_APPEND=0: rotate q, rotate k and append to the cache as three launches instead of one
        self.fused_rope_append = os.environ.get("VERL_B200_FUSED_ROPE_APPEND", "1") != "0"
        self.grouped_decode = (self.is_cuda and self.share_prefill and self.bs == 64 and self.cfg.head_dim in (64, 128)
                               and nh_l // max(1, nkv_l) <= 16 and os.environ.get("VERL_B200_GROUPED_DECODE", "0") == "1")
        self._groups: dict[int, list[int]] = {}
        self._slot_group: dict[int, int] = {}
        self._free_gids = list(range(S - 1, -1, -1))
        if self.grouped_decode:
            self.grp_members = torch.full((S, 8), -1, dtype=torch.int32, device=dev)
            self.grp_pages = torch.zeros(S, dtype=torch.int32, device=dev)
            self.seq_skip = torch.zeros(S, dtype=torch.int32, device=dev)
            self.pd_splits = (2, 1 if S * nkv_l >= 296 else min(8, -(-296 // (S * nkv_l))))
            self.pd_ws = torch.empty(S * nh_l * sum(self.pd_splits) * (self.cfg.head_dim + 2), dtype=torch.float32, device=dev)

    # ------------------------------------------------------------------------------------ decode groups
    def _form_groups(self, reqs: list, leaders: list[int], lead_idx: list[int], lens: list[int]) -> None:
        """After a prefill wave: the requests that share a leader's prompt pages become decode groups of up to 8 members."""
        if not self.grouped_decode:
            return
        by_leader: dict[int, list[int]] = {}
        for i, r in enumerate(reqs):
            by_leader.setdefault(lead_idx[i], []).append(i)
        for j, idxs in by_leader.items():
            nfull = lens[leaders[j]] // self.bs
            if len(idxs) < 2 or nfull == 0:
                continue
            for c0 in range(0, len(idxs), 8):
                part = idxs[c0 : c0 + 8]
                if len(part) < 2 or not self._free_gids:
                    continue
                gid = self._free_gids.pop()
                slots = [reqs[i].slot for i in part]
                self._groups[gid] = slots
                for sl in slots:
                    self._slot_group[sl] = gid
                self._write_group(gid, nfull)

    def _write_group(self, gid: int, pages: Optional[int] = None) -> None:
        slots = self._groups.get(gid, [])
        row = torch.full((8,), -1, dtype=torch.int32)
        row[: len(slots)] = torch.tensor(slots, dtype=torch.int32)
        self.grp_members[gid] = row.to(self.device)
        if pages is not None:
            self.grp_pages[gid] = pages
            self.seq_skip[torch.tensor(slots, dtype=torch.int64, device=self.device)] = pages

    def _leave_group(self, slot: int) -> None:
        """A sequence's slot is released: it leaves its group; a group of one is dissolved (nothing left to share)."""
        gid = self._slot_group.pop(slot, None)
        if gid is None:
            return
        self.seq_skip[slot] = 0
        members = self._groups[gid]
        members.remove(slot)
        if len(members) < 2:
            for sl in members:
                self._slot_group.pop(sl, None)
                self.seq_skip[sl] = 0
            self._groups.pop(gid)
            self.grp_pages[gid] = 0
            self.grp_members[gid] = -1
            self._free_gids.append(gid)
        else:
            self._write_group(gid)

    def _ensure_out(self, cap: int) -> None:
        if cap > self.out_cap:
            assert not self.running, "output capacity can only grow while idle"
            self.out_cap = int(cap)
            self.out_tok = torch.zeros(self.S, self.out_cap, dtype=torch.int64, device=self.device)
            self.out_lp = torch.zeros(self.S, self.out_cap, dtype=torch.float32, device=self.device)
            if self.record_routing:
                self.out_routed = torch.zeros(self.S, self.out_cap, self.cfg.num_hidden_layers, self.cfg.num_experts_per_tok,
                                              dtype=torch.int16, device=self.device)
            self._graph = None

    # ------------------------------------------------------------------------------------ requests
    def add_request(self, prompt_ids: Sequence[int], params: SamplingParams, request_id: Optional[str] = None) -> str:
        rid = request_id if request_id is not None else f"req-{self._rid}"
        self._rid += 1
        prompt = list(map(int, prompt_ids))
        assert 0 < len(prompt) < self.max_model_len, f"prompt of {len(prompt)} tokens does not fit max_model_len"
        p = SamplingParams(**{**params.__dict__})
        p.max_tokens = max(1, min(p.max_tokens, self.max_model_len - len(prompt)))
        self.waiting.append(_Request(rid, prompt, p, arrival=time.time()))
        return rid

    def abort(self, request_id: Optional[str] = None) -> list[RequestOutput]:
        """Abort one request (or all): running sequences are retired with what they generated so far."""
        out = []
        if self.running:
            self._sync_retire(force_rids=None if request_id is None else {request_id}, abort=True)
        keep = deque()
        for r in self.waiting:
            if request_id is None or r.rid == request_id:
                out.append(RequestOutput(r.rid, r.prompt, [], [], "aborted"))
            else:
                keep.append(r)
        self.waiting = keep
        self.finished.extend(out)
        return out

    def has_unfinished(self) -> bool:
        return bool(self.waiting or self.running)

    # ------------------------------------------------------------------------------------ prefill
    def _prefill_kv_hook(self, layer: int, k: torch.Tensor, v: torch.Tensor) -> None:
        if self._prefill_slots is not None:
            F.kv_append_(k, v, self._prefill_slots, self.kv[layer, 0], self.kv[layer, 1])

    _prefill_slots: Optional[torch.Tensor] = None

    def _admit(self) -> list[_Request]:
        """Move waiting requests into free slots while blocks and the token budget last."""
        batch, tokens = [], 0
        while self.waiting and self.free_slots:
            r = self.waiting[0]
            need = (len(r.prompt) + r.params.max_tokens + self.bs - 1) // self.bs
            hit: list[int] = []
            if self.enable_prefix_caching and r.handoff is None:
                # longest run of leading pages that is in the cache; the last prompt token is always computed (its output
                # is the first sampling distribution)
                for h in self._page_hashes(r.prompt, (len(r.prompt) - 1) // self.bs):
                    b = self._page_of_hash.get(h)
                    if b is None:
                        break
                    hit.append(b)
            idle_hit = sum(1 for b in hit if b in self._idle_cached)
            if need - len(hit) > len(self.free_blocks) + len(self._idle_cached) - idle_hit or \
                    (batch and tokens + len(r.prompt) - len(hit) * self.bs > self.max_batched):
                break
            want = (r.params.temperature, r.params.top_k, r.params.top_p)
            idle = not self.running and not batch
            if idle:
                self.temperature, self.top_k, self.top_p = want  # one sampling configuration per running wave
                self._ensure_out(r.params.max_tokens)
            elif want != (self.temperature, self.top_k, self.top_p) or r.params.max_tokens > self.out_cap:
                break
            self.waiting.popleft()
            r.slot = self.free_slots.pop()
            for b in hit:                       # cached pages gain a user
                if b in self._idle_cached:
                    del self._idle_cached[b]
                else:
                    self._block_users[b] = self._block_users.get(b, 1) + 1
            r.cached = len(hit) * self.bs
            r.blocks = hit + [self._take_block() for _ in range(need - len(hit))]
            batch.append(r)
            tokens += len(r.prompt) - r.cached
        return batch

    # ------------------------------------------------------------------------------------ prefill / decode disaggregation
    @torch.no_grad()
    def prefill_only(self, prompts: Sequence[Sequence[int]], params: SamplingParams | Sequence[SamplingParams]) -> list[dict]:
        """Prefill stage of a disaggregated deployment: run the prompts, sample the first token, and hand back per prompt
        what a decode engine needs to continue (``add_prefilled``): the KV content of the prompt's pages, the first token
        with its log-prob and the sampler state. Nothing stays allocated here afterwards."""
        plist = list(params) if isinstance(params, (list, tuple)) else [params] * len(prompts)
        assert not self.running and not self.waiting, "prefill_only needs an idle engine"
        self._ensure_out(max(p.max_tokens for p in plist))
        rids = [self.add_request(p, sp) for p, sp in zip(prompts, plist)]
        out: dict[str, dict] = {}
        while self.waiting:
            reqs = self._admit()
            assert reqs, "a prompt does not fit the prefill engine's cache"
            self._prefill(reqs)
            for r in reqs:
                nb = (len(r.prompt) + self.bs - 1) // self.bs
                blk = torch.tensor(r.blocks[:nb], dtype=torch.int64, device=self.device)
                out[r.rid] = dict(prompt=list(r.prompt), kv=self.kv[:, :, blk].clone(), token=int(self.tok[r.slot]),
                                  logprob=float(self.out_lp[r.slot, 0]), seed=int(self.seeds[r.slot]), block_size=self.bs,
                                  routed_prompt=getattr(r, "routed_prompt", None))
            idx = torch.tensor([r.slot for r in reqs], dtype=torch.int64, device=self.device)
            for r in reqs:
                self.running.pop(r.slot)
                self._leave_group(r.slot)
                self._release_blocks(r.blocks)
                self.free_slots.append(r.slot)
            self.active[idx] = False
            self.ctx[idx] = 0
        return [out[r] for r in rids]

    def add_prefilled(self, handoff: dict, params: SamplingParams, request_id: Optional[str] = None) -> str:
        """Decode stage: queue a request whose prompt was prefilled by another engine (same model, same block size)."""
        assert handoff["block_size"] == self.bs, "prefill and decode engines must use the same KV block size"
        rid = self.add_request(handoff["prompt"], params, request_id)
        self.waiting[-1].handoff = handoff
        return rid

    @torch.no_grad()
    def _install_prefilled(self, reqs: list[_Request]) -> None:
        dev = self.device
        lens = [len(r.prompt) for r in reqs]
        bt_rows = torch.zeros(len(reqs), self.max_blocks_per_seq, dtype=torch.int32)
        for i, r in enumerate(reqs):
            bt_rows[i, : len(r.blocks)] = torch.tensor(r.blocks, dtype=torch.int32)
            nb = (lens[i] + self.bs - 1) // self.bs
            dst = torch.tensor(r.blocks[:nb], dtype=torch.int64, device=dev)
            self.kv[:, :, dst] = r.handoff["kv"].to(dev, dtype=self.kv.dtype)   # the KV transfer (a peer copy between GPUs)
            if self.record_routing:
                r.routed_prompt = r.handoff.get("routed_prompt")
        slots = torch.tensor([r.slot for r in reqs], dtype=torch.int64, device=dev)
        tok = torch.tensor([r.handoff["token"] for r in reqs], dtype=torch.int64, device=dev)
        lp = torch.tensor([r.handoff["logprob"] for r in reqs], dtype=torch.float32, device=dev)
        stop_rows = torch.full((len(reqs), 8), -1, dtype=torch.int64)
        for i, r in enumerate(reqs):
            st = list(r.params.stop_token_ids or ())[:8]
            if st:
                stop_rows[i, : len(st)] = torch.tensor(st, dtype=torch.int64)
        self.stop_ids[slots] = stop_rows.to(dev)
        pens = [float(r.params.repetition_penalty or 1.0) for r in reqs]
        if any(p != 1.0 for p in pens) and not self._use_penalty:
            self.seen = torch.zeros(self.S, self.cfg.vocab_size, dtype=torch.bool, device=dev)
            self._use_penalty, self._graph = True, None
        self.rep_penalty[slots] = torch.tensor(pens, dtype=torch.float32, device=dev)
        if self._use_penalty:
            self.seen[slots] = False
            for r in reqs:
                self.seen[r.slot, torch.tensor(r.prompt + [r.handoff["token"]], dtype=torch.int64, device=dev)] = True
        n = torch.tensor(lens, dtype=torch.int32, device=dev)
        self.block_table[slots] = bt_rows.to(dev)
        self.tok[slots] = tok
        self.pos[slots] = n
        self.ctx[slots] = n + 1
        self.gen[slots] = 1
        self.max_new[slots] = torch.tensor([r.params.max_tokens for r in reqs], dtype=torch.int32, device=dev)
        self.ignore_eos[slots] = torch.tensor([r.params.ignore_eos for r in reqs], dtype=torch.bool, device=dev)
        self.seeds[slots] = torch.tensor([r.handoff["seed"] for r in reqs], dtype=torch.int64, device=dev)
        self.out_tok[slots, 0] = tok
        self.out_lp[slots, 0] = lp
        done = (self.gen[slots] >= self.max_new[slots])
        if self.eos is not None:
            done |= (tok == self.eos) & ~self.ignore_eos[slots]
        done |= (tok.unsqueeze(1) == self.stop_ids[slots]).any(1)
        self.active[slots] = ~done
        for r in reqs:
            self.running[r.slot] = r

    @torch.no_grad()
    def _prefill(self, reqs: list[_Request]) -> None:
        hand = [r for r in reqs if r.handoff is not None]
        if hand:
            self._install_prefilled(hand)
            reqs = [r for r in reqs if r.handoff is None]
            if not reqs:
                return
        t0 = time.time()
        dev = self.device
        lens = [len(r.prompt) for r in reqs]
        # requests with the same prompt (the n samples of a group) are prefilled once: the leader's prompt runs through
        # the model, the followers get a copy of its KV blocks and sample their own first token from the same logits
        first_of: dict = {}
        leaders: list[int] = []   # request index of each distinct prompt's first occurrence
        lead_idx: list[int] = []  # per request: index into ``leaders``
        for i, r in enumerate(reqs):
            key = tuple(r.prompt) if self.share_prefill else i
            if key not in first_of:
                first_of[key] = len(leaders)
                leaders.append(i)
            lead_idx.append(first_of[key])
        # followers point at the leader's pages for every page the prompt fills completely (those are never written
        # again); decode CTAs of a group then stream the same addresses at the same time and meet in L2
        if len(leaders) < len(reqs):
            for i, r in enumerate(reqs):
                li = leaders[lead_idx[i]]
                nfull = lens[i] // self.bs
                if li == i or nfull == 0:
                    continue
                own, shared = r.blocks[:nfull], reqs[li].blocks[:nfull]
                self._release_blocks(own)
                r.blocks[:nfull] = shared
                for b in shared:
                    self._block_users[b] = self._block_users.get(b, 1) + 1
        bt_rows = torch.zeros(len(reqs), self.max_blocks_per_seq, dtype=torch.int32)
        for i, r in enumerate(reqs):
            bt_rows[i, : len(r.blocks)] = torch.tensor(r.blocks, dtype=torch.int32)
        skip = [reqs[i].cached for i in leaders]        # tokens whose pages came from the prefix cache: not recomputed
        ids = torch.tensor([t for i in leaders for t in reqs[i].prompt[reqs[i].cached:]], dtype=torch.int64)
        slot_rows = []
        for i in leaders:
            p = torch.arange(reqs[i].cached, lens[i])
            slot_rows.append(bt_rows[i, p // self.bs].long() * self.bs + p % self.bs)
        if self.is_cuda:
            ids, slot_map = ids.pin_memory().to(dev, non_blocking=True), torch.cat(slot_rows).pin_memory().to(dev, non_blocking=True)
        else:
            slot_map = torch.cat(slot_rows)
        batch = PackedBatch.from_lengths(ids, [lens[i] - c for i, c in zip(leaders, skip)], device=dev)
        if any(skip):
            batch.positions = torch.cat([torch.arange(c, lens[i], dtype=torch.int32) for i, c in zip(leaders, skip)]).to(dev)
            pages = torch.cat([bt_rows[i, : c // self.bs].long() for i, c in zip(leaders, skip)])
            cached_slots = (pages.unsqueeze(1) * self.bs + torch.arange(self.bs).unsqueeze(0)).reshape(-1).to(dev)
            nkv_l, hd = self.kv.shape[-2], self.kv.shape[-1]
            self.model.prefix_kv = lambda layer: (self.kv[layer, 0].view(-1, nkv_l, hd)[cached_slots],
                                                  self.kv[layer, 1].view(-1, nkv_l, hd)[cached_slots], skip)
            self.model._ensure_rope(max(lens) + 1)
            self.stats["prefix_cache_hit_tokens"] = self.stats.get("prefix_cache_hit_tokens", 0) + sum(skip)
        self._prefill_slots = slot_map
        if self.record_routing:
            from ....models.decoder import RouterReplay

            self.model.router_replay = RouterReplay("record")
        try:
            h = self.model.forward_hidden(batch)
        finally:
            self._prefill_slots = None
            self.model.prefix_kv = None
        if self.enable_prefix_caching:
            for i in leaders:
                self._index_pages(reqs[i].prompt, reqs[i].blocks, lens[i])
        if self.record_routing:
            routed = self.model.router_replay.stacked(list(range(self.cfg.num_hidden_layers))).to(torch.int16).cpu()
            self.model.router_replay = None
            cu = [0]
            for i in leaders:
                cu.append(cu[-1] + lens[i])
            for i, r in enumerate(reqs):
                j = lead_idx[i]
                r.routed_prompt = routed[cu[j] : cu[j + 1]]
        last = (batch.cu_seqlens[1:].long() - 1)
        logits = F.gemm(h[last].contiguous(), self.params.lm_head_weight)
        if len(leaders) < len(reqs):
            logits = logits[torch.tensor(lead_idx, dtype=torch.int64, device=dev)]
            for i, r in enumerate(reqs):
                li = leaders[lead_idx[i]]
                if li == i:
                    continue
                nfull, nb = lens[i] // self.bs, (lens[i] + self.bs - 1) // self.bs
                if nb > nfull:  # the partially filled last page is private: copy it
                    src = torch.tensor(reqs[li].blocks[nfull:nb], dtype=torch.int64, device=dev)
                    dst = torch.tensor(r.blocks[nfull:nb], dtype=torch.int64, device=dev)
                    self.kv[:, :, dst] = self.kv[:, :, src]
            self.stats["prefill_tokens_shared"] = self.stats.get("prefill_tokens_shared", 0) + sum(lens) - sum(lens[i] for i in leaders)
        slots = torch.tensor([r.slot for r in reqs], dtype=torch.int64, device=dev)
        seeds = torch.tensor([(r.params.seed if r.params.seed is not None else self._seed * 1000003 + zlib.crc32(r.rid.encode()))
                              for r in reqs], dtype=torch.int64, device=dev)
        stop_rows = torch.full((len(reqs), 8), -1, dtype=torch.int64)
        for i, r in enumerate(reqs):
            st = list(r.params.stop_token_ids or ())[:8]
            if st:
                stop_rows[i, : len(st)] = torch.tensor(st, dtype=torch.int64)
        self.stop_ids[slots] = stop_rows.to(dev)
        pens = [float(r.params.repetition_penalty or 1.0) for r in reqs]
        if any(p != 1.0 for p in pens) and not self._use_penalty:
            self.seen = torch.zeros(self.S, self.cfg.vocab_size, dtype=torch.bool, device=dev)
            self._use_penalty, self._graph = True, None  # the decode graph gains the penalty ops
        self.rep_penalty[slots] = torch.tensor(pens, dtype=torch.float32, device=dev)
        if self._use_penalty:
            self.seen[slots] = False
            for i, r in enumerate(reqs):
                self.seen[r.slot, torch.tensor(r.prompt, dtype=torch.int64, device=dev)] = True
            logits = self._penalise(logits, slots)
        tok, lp = F.sample_tokens(logits, self.temperature, seeds, 0, self.valid_vocab, self.top_k, self.top_p)
        if self._use_penalty:
            self.seen[slots, tok] = True
        n = torch.tensor(lens, dtype=torch.int32, device=dev)
        self.block_table[slots] = bt_rows.to(dev)
        if len(leaders) < len(reqs):
            self._form_groups(reqs, leaders, lead_idx, lens)
        self.tok[slots] = tok
        self.pos[slots] = n
        self.ctx[slots] = n + 1
        self.gen[slots] = 1
        self.max_new[slots] = torch.tensor([r.params.max_tokens for r in reqs], dtype=torch.int32, device=dev)
        self.ignore_eos[slots] = torch.tensor([r.params.ignore_eos for r in reqs], dtype=torch.bool, device=dev)
        self.seeds[slots] = seeds * 6364136223846793005 + 1442695040888963407
        self.out_tok[slots, 0] = tok
        self.out_lp[slots, 0] = lp
        done = (self.gen[slots] >= self.max_new[slots])
        if self.eos is not None:
            done |= (tok == self.eos) & ~self.ignore_eos[slots]
        done |= (tok.unsqueeze(1) == self.stop_ids[slots]).any(1)
        self.active[slots] = ~done
        for r in reqs:
            self.running[r.slot] = r
        self.stats["prefill_tokens"] += sum(lens) - sum(skip)
        self.stats["prefill_s"] += time.time() - t0

    def _penalise(self, logits: torch.Tensor, slots=None) -> torch.Tensor:
        """Repetition penalty: logits of tokens that already occur in a sequence are divided (positive) or multiplied
        (negative) by the sequence's penalty."""
        seen = self.seen if slots is None else self.seen[slots]
        pen = (self.rep_penalty if slots is None else self.rep_penalty[slots]).unsqueeze(1)
        l = logits.float()
        V = min(l.shape[1], seen.shape[1])
        l[:, :V] = torch.where(seen[:, :V], torch.where(l[:, :V] > 0, l[:, :V] / pen, l[:, :V] * pen), l[:, :V])
        return l.to(logits.dtype)

    # ------------------------------------------------------------------------------------ decode
    def _decode_body(self) -> None:
        """One decode step over all slots (static shapes; capturable)."""
        cfg, P = self.cfg, self.params
        S = self.S
        act = self.active
        acti = act.to(torch.int32)
        pos_l = self.pos.long()
        blk = torch.gather(self.block_table, 1, (pos_l // self.bs).unsqueeze(1)).squeeze(1).long()
        slot_map = torch.where(act, blk * self.bs + pos_l % self.bs, torch.full_like(pos_l, -1))
        ctx_eff = self.ctx * acti
        tp = self.model.tp
        w_ = self.tp_size
        nh, nkv, hd, Q, KV = cfg.num_attention_heads // w_, cfg.num_key_value_heads // w_, cfg.head_dim, cfg.q_size // w_, cfg.kv_size // w_
        a = F.embedding(self.tok, P["embed_tokens.weight"])
        r = None
        cos, sin = self.model._cos, self.model._sin
        pd_groups = (self.grp_members, self.grp_pages, self.seq_skip, self.pd_ws, *self.pd_splits) if self.grouped_decode else None
        if self.record_routing:
            from ....models.decoder import RouterReplay

            self.model.router_replay = RouterReplay("record")
        for i in range(cfg.num_hidden_layers):
            W = P.layer(i)
            self.model._layer_idx = i
            h1, x, _ = F.rms_norm(a, W["input_layernorm.weight"], cfg.rms_norm_eps, residual=r)
            if tp is not None:
                qkv = self.model.qkv_tp(W, h1)
            else:
                qkv = self.model._lin(W, "self_attn.qkv_proj.weight", h1)
            q = qkv[:, :Q].view(S, nh, hd)
            k = qkv[:, Q : Q + KV].view(S, nkv, hd)
            v = qkv[:, Q + KV :].view(S, nkv, hd)
            if cfg.qk_norm:
                qn = F.rms_norm(q.reshape(S * nh, hd).contiguous(), W["self_attn.q_norm.weight"], cfg.rms_norm_eps)[0]
                kn = F.rms_norm(k.reshape(S * nkv, hd).contiguous(), W["self_attn.k_norm.weight"], cfg.rms_norm_eps)[0]
                q.copy_(qn.view(S, nh, hd))
                k.copy_(kn.view(S, nkv, hd))
            if cfg.qk_norm or not qkv.is_contiguous() or not self.fused_rope_append:
                F.apply_rope_(q, self.pos, cos, sin)
                F.apply_rope_(k, self.pos, cos, sin)
                F.kv_append_(k, v, slot_map, self.kv[i, 0], self.kv[i, 1])
            else:  # one launch: rotate q and k in the projection output, append k and v to the cache
                F.rope_kv_append_(qkv, self.pos, cos, sin, slot_map, self.kv[i, 0], self.kv[i, 1], nh, nkv, hd)
            attn = F.paged_decode_attention(q, self.kv[i, 0], self.kv[i, 1], self.block_table, ctx_eff, groups=pd_groups)
            if tp is not None:
                o = tp.row_linear(attn.reshape(S, Q), W["self_attn.o_proj.weight"][:, tp.rows(cfg.q_size)], None)
            else:
                o = self.model._lin(W, "self_attn.o_proj.weight", attn.reshape(S, Q))
            h2, x2, _ = F.rms_norm(o, W["post_attention_layernorm.weight"], cfg.rms_norm_eps, residual=x)
            a = self.model._mlp_fwd(W, h2, None)
            r = x2
        hN = F.rms_norm(a, P["norm.weight"], cfg.rms_norm_eps, residual=r)[0]
        if tp is not None and self._tp_share is not None and not self._use_penalty:
            sh = S // tp.size
            mine = slice(tp.rank * sh, (tp.rank + 1) * sh)
            logits = F.gemm(hN[mine], P.lm_head_weight)
            tok_h, lp_h = F.sample_tokens(logits, self.temperature, self.seeds[mine].contiguous(), 0, self.valid_vocab, self.top_k, self.top_p)
            both = self._tp_share(torch.cat([tok_h.to(torch.int32), lp_h.float().view(torch.int32)]))   # [tp, 2 * sh]
            tok = both[:, :sh].reshape(S).long()
            lp = both[:, sh:].reshape(S).view(torch.float32)
        else:
            logits = F.gemm(hN, P.lm_head_weight)
            if self._use_penalty:
                logits = self._penalise(logits)
            tok, lp = F.sample_tokens(logits, self.temperature, self.seeds, 0, self.valid_vocab, self.top_k, self.top_p)
        # ---- state update (all on device)
        rows = torch.arange(S, device=self.device)
        if self.record_routing:
            # routing of the token that was fed in this step = generated token number gen - 1
            step_routed = self.model.router_replay.stacked(list(range(cfg.num_hidden_layers))).to(torch.int16)
            self.model.router_replay = None
            prev = (self.gen.long() - 1).clamp(min=0, max=self.out_cap - 1)
            self.out_routed[rows, prev] = torch.where(act.view(-1, 1, 1), step_routed, self.out_routed[rows, prev])
        if self._use_penalty:
            self.seen[rows, tok] = self.seen[rows, tok] | act
        col = self.gen.long().clamp(max=self.out_cap - 1)
        self.out_tok[rows, col] = torch.where(act, tok, self.out_tok[rows, col])
        self.out_lp[rows, col] = torch.where(act, lp, self.out_lp[rows, col])
        self.gen.add_(acti)
        done = self.gen >= self.max_new
        if self.eos is not None:
            done = done | ((tok == self.eos) & ~self.ignore_eos)
        done = done | (tok.unsqueeze(1) == self.stop_ids).any(1)
        self.tok.copy_(torch.where(act, tok, self.tok))
        self.pos.add_(acti)
        self.ctx.add_(acti)
        self.active.copy_(act & ~done)
        self.seeds.copy_(self.seeds * 6364136223846793005 + 1442695040888963407)

    @torch.no_grad()
    def _decode_steps(self, n: int) -> None:
        t0 = time.time()
        ev = None
        if self.is_cuda:  # device time of the decode steps, read at the next host synchronisation (``_sync_retire``)
            ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            ev[0].record()
        if not self.use_graph or self.cfg.is_moe:
            for _ in range(n):
                self._decode_body()
        else:
            key = (self.temperature, self.top_k, self.top_p, self.out_cap, id(self.kv))
            if self._graph is None or self._graph_key != key:
                snap = [t.clone() for t in (self.tok, self.pos, self.ctx, self.gen, self.active, self.seeds, self.out_tok, self.out_lp)]
                side = torch.cuda.Stream(device=self.device)
                side.wait_stream(torch.cuda.current_stream(self.device))
                with torch.cuda.stream(side):
                    self._decode_body()  # warm-up (allocator, lazy init) outside capture
                torch.cuda.current_stream(self.device).wait_stream(side)
                for dst, src in zip((self.tok, self.pos, self.ctx, self.gen, self.active, self.seeds, self.out_tok, self.out_lp), snap):
                    dst.copy_(src)
                from ....ops import native

                g = torch.cuda.CUDAGraph()
                n0 = native.launch_count()
                with torch.cuda.graph(g):
                    self._decode_body()
                self._graph_kernels = native.launch_count() - n0
                native.add_launches(-self._graph_kernels)  # captured, not launched
                for dst, src in zip((self.tok, self.pos, self.ctx, self.gen, self.active, self.seeds, self.out_tok, self.out_lp), snap):
                    dst.copy_(src)
                self._graph, self._graph_key = g, key
            for _ in range(n):
                self._graph.replay()
            from ....ops import native

            native.add_launches(self._graph_kernels * n)
        if ev is not None:
            ev[1].record()
            self._decode_events.append(ev)
        self.stats["decode_steps"] += n
        self.stats["decode_s"] += time.time() - t0

    # ------------------------------------------------------------------------------------ retire
    def _sync_retire(self, force_rids=None, abort: bool = False) -> None:
        if not self.running:
            return
        active = self.active.cpu()
        gen = self.gen.cpu()
        if self._decode_events:
            self._decode_events[-1][1].synchronize()
            self.stats["decode_gpu_s"] = self.stats.get("decode_gpu_s", 0.0) + sum(a.elapsed_time(b) for a, b in self._decode_events) * 1e-3
            self._decode_events.clear()
        done_slots = [s for s, r in self.running.items()
                      if (not bool(active[s])) or (abort and (force_rids is None or r.rid in force_rids))]
        if not done_slots:
            return
        idx = torch.tensor(done_slots, dtype=torch.int64, device=self.device)
        toks = self.out_tok[idx].cpu()
        lps = self.out_lp[idx].cpu()
        routed = self.out_routed[idx].cpu() if self.record_routing else None
        for j, s in enumerate(done_slots):
            r = self.running.pop(s)
            n = int(gen[s])
            t = toks[j, :n].tolist()
            still_active = bool(active[s])
            if still_active:
                reason = "aborted"
            elif n > 0 and ((self.eos is not None and t[-1] == self.eos and not r.params.ignore_eos)
                            or t[-1] in tuple(r.params.stop_token_ids or ())):
                reason = "completed"
            else:
                reason = "length"
            extra = {}
            if routed is not None:
                # prompt tokens, then every generated token that was fed back (all but the last one)
                extra["routed_experts"] = torch.cat([r.routed_prompt, routed[j, : max(n - 1, 0)]], 0)
            self.finished.append(RequestOutput(r.rid, r.prompt, t, lps[j, :n].tolist() if r.params.logprobs else None, reason,
                                               extra_fields=extra))
            self.stats["generated_tokens"] += n
            if self.enable_prefix_caching and n > 1:
                # the next turn of a conversation starts with this prompt + response: every generated token but the last
                # has gone through the model, its keys / values are in the pages
                self._index_pages(r.prompt + t[:-1], r.blocks, len(r.prompt) + n - 1)
            self._leave_group(s)
            self._release_blocks(r.blocks)
            self.free_slots.append(s)
        self.active[idx] = False
        self.ctx[idx] = 0

    # ------------------------------------------------------------------------------------ driver loops
    def step(self) -> list[RequestOutput]:
        """Admit + prefill what fits, run ``sync_interval`` decode steps, retire; returns newly finished."""
        assert self.kv is not None, "KV cache released; call resume_kv_cache() first"
        if self.waiting and not self.running:
            self._ensure_out(max(r.params.max_tokens for r in self.waiting))
        while True:
            reqs = self._admit()
            if not reqs:
                break
            self._prefill(reqs)
        if self.running:
            self._decode_steps(self.sync_interval)
            self._sync_retire()
        out, self.finished = self.finished, []
        return out

    def generate(self, prompts: Sequence[Sequence[int]], params: SamplingParams | Sequence[SamplingParams]) -> list[RequestOutput]:
        """Blocking batch generation; outputs are returned in prompt order."""
        plist = list(params) if isinstance(params, (list, tuple)) else [params] * len(prompts)
        if not self.running:
            self._ensure_out(max(p.max_tokens for p in plist))
        rids = [self.add_request(p, sp) for p, sp in zip(prompts, plist)]
        results: dict[str, RequestOutput] = {}
        while len(results) < len(rids):
            progressed = self.step()
            for o in progressed:
                results[o.request_id] = o
            if not progressed and not self.has_unfinished():
                break
        return [results[r] for r in rids]
