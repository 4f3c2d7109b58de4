"""Shared-prefix ("prefix grouper") utilities: the n samples of a prompt share its tokens in the token-wise layers of the
log-prob and training passes, and only attention sees one full sequence per sample.

The packing itself lives next to the engine (``workers/engine/native/engine.py``: ``prompt_group_ids``,
``pack_shared_prefix_batch``; the decoder expands / collapses around attention with ``PackedBatch.expand_index`` /
``collapse_index``). This module is the trainer-facing surface: group detection, the position ids of a grouped stream,
the token savings of a batch, and a forward over a micro-batch with sharing switched on.

Parity target: ``verl/trainer/ppo/prefix_grouper_utils.py`` (``build_position_ids_for_prefix_grouper`` :23,
``build_pg_from_micro_batch`` :46, ``pg_forward`` :103, ``forward_micro_batch_with_prefix_grouper`` :150).
"""

from __future__ import annotations

from typing import Optional

import torch

from ...workers.engine.native.engine import pack_shared_prefix_batch, prompt_group_ids

__all__ = ["prompt_group_ids", "pack_shared_prefix_batch", "build_pg_from_micro_batch", "build_position_ids_for_prefix_grouper",
           "shared_prefix_token_savings", "forward_micro_batch_with_prefix_grouper"]


def build_pg_from_micro_batch(micro_batch: dict, response_length: Optional[int] = None) -> dict:
    """Group structure of a padded micro-batch (left-padded prompts, right-padded responses): per group the row indices,
    the prompt length and the response lengths."""
    ids, am = micro_batch["input_ids"], micro_batch["attention_mask"]
    R = int(response_length if response_length is not None else micro_batch["responses"].shape[1])
    P = ids.shape[1] - R
    gids = prompt_group_ids(ids, am, R)
    plen, rlen = am[:, :P].sum(-1).tolist(), am[:, P:].sum(-1).tolist()
    groups: list[dict] = []
    for row, g in enumerate(gids):
        if not groups or groups[-1]["gid"] != g:
            groups.append({"gid": g, "rows": [], "prefix_len": int(plen[row]), "suffix_lens": []})
        groups[-1]["rows"].append(row)
        groups[-1]["suffix_lens"].append(int(rlen[row]))
    return {"gids": gids, "groups": groups, "response_length": R}


def build_position_ids_for_prefix_grouper(pg: dict) -> torch.Tensor:
    """Positions of the grouped stream: the shared prompt counts 0..p-1 once, every response continues at p."""
    out = []
    for g in pg["groups"]:
        p = g["prefix_len"]
        out.append(torch.arange(p))
        out += [torch.arange(p, p + r) for r in g["suffix_lens"]]
    return torch.cat(out) if out else torch.zeros(0, dtype=torch.int64)


def shared_prefix_token_savings(pg: dict) -> tuple[int, int]:
    """(tokens with one prompt copy per group, tokens with one per sample)."""
    shared = sum(g["prefix_len"] + sum(g["suffix_lens"]) for g in pg["groups"])
    plain = sum(g["prefix_len"] * len(g["rows"]) + sum(g["suffix_lens"]) for g in pg["groups"])
    return shared, plain


def forward_micro_batch_with_prefix_grouper(engine, micro_batch: dict, temperature: float = 1.0, calculate_entropy: bool = False) -> dict:
    """Log-probs (and entropy) of the responses of one micro-batch with the prompts shared inside their groups."""
    R = micro_batch["responses"].shape[1]
    mb = dict(micro_batch)
    mb.setdefault("_rows", list(range(mb["input_ids"].shape[0])))
    mb["_gids"] = prompt_group_ids(mb["input_ids"], mb["attention_mask"], R)
    with torch.no_grad():
        return engine._forward_micro(mb, R, temperature, calculate_entropy, need_grad=False)
