"""Training metrics: data statistics, timing, throughput, validation aggregation.

Parity target: ``verl/trainer/ppo/metric_utils.py`` (``compute_data_metrics`` :429, ``compute_timing_metrics`` :611,
``compute_throughout_metrics`` :655-688, ``process_validation_metrics`` :896).
"""

from __future__ import annotations

from collections import defaultdict
from functools import partial
from typing import Any, Callable

import numpy as np
import torch

from ...protocol import DataProto
from ...utils import torch_functional as VF

__all__ = ["reduce_metrics", "compute_data_metrics", "compute_timing_metrics", "compute_throughout_metrics",
           "compute_variance_proxy_metrics", "bootstrap_metric", "calc_maj_val", "process_validation_metrics",
           "_compute_response_info"]


def _flatten(v):
    """Leaves of arbitrarily nested lists/tuples/arrays (per-worker lists of per-micro-batch lists)."""
    if isinstance(v, np.ndarray):
        v = v.reshape(-1).tolist()
    for x in v:
        if isinstance(x, (list, tuple, np.ndarray)):
            yield from _flatten(x)
        else:
            yield x


def reduce_metrics(metrics: dict[str, Any]) -> dict[str, float]:
    """Mean of list-valued metrics; keys containing 'max'/'min' reduce with max/min."""
    out = {}
    for k, v in metrics.items():
        if isinstance(v, (list, tuple, np.ndarray)):
            vals = [float(x) for x in _flatten(v)]
            if not vals:
                continue
            out[k] = float(np.max(vals)) if "max" in k.split("/")[-1] else float(np.min(vals)) if "min" in k.split("/")[-1] else float(np.mean(vals))
        else:
            out[k] = float(v)
    return out


def _compute_response_info(batch: DataProto) -> dict[str, Any]:
    R = batch.batch["responses"].shape[-1]
    am = batch.batch["attention_mask"]
    prompt_mask, response_mask = am[:, :-R], am[:, -R:]
    if "response_mask" in batch.batch.keys():
        response_mask = batch.batch["response_mask"]
    return dict(response_mask=response_mask, prompt_length=prompt_mask.sum(-1).float(),
                response_length=response_mask.sum(-1).float())


def _stats(prefix: str, t: torch.Tensor) -> dict[str, float]:
    return {f"{prefix}/mean": t.mean().item(), f"{prefix}/max": t.max().item(), f"{prefix}/min": t.min().item()}


def compute_data_metrics(batch: DataProto, use_critic: bool = True) -> dict[str, Any]:
    seq_score = batch.batch["token_level_scores"].sum(-1)
    seq_reward = batch.batch["token_level_rewards"].sum(-1)
    adv, ret = batch.batch["advantages"], batch.batch["returns"]
    info = _compute_response_info(batch)
    mask = info["response_mask"].bool()
    R = batch.batch["responses"].shape[-1]
    P = batch.batch["attention_mask"].shape[-1] - R
    resp_len, prompt_len = info["response_length"], info["prompt_length"]
    aborted = resp_len == 0
    nz = ~aborted
    m = {}
    m.update({f"critic/score/{k.split('/')[-1]}": v for k, v in _stats("x", seq_score).items()})
    m.update({f"critic/rewards/{k.split('/')[-1]}": v for k, v in _stats("x", seq_reward).items()})
    if mask.any():
        m.update({f"critic/advantages/{k.split('/')[-1]}": v for k, v in _stats("x", adv[mask]).items()})
        m.update({f"critic/returns/{k.split('/')[-1]}": v for k, v in _stats("x", ret[mask]).items()})
    if use_critic and "values" in batch.batch.keys() and mask.any():
        vals = batch.batch["values"]
        m.update({f"critic/values/{k.split('/')[-1]}": v for k, v in _stats("x", vals[mask]).items()})
        var_ret = torch.var(ret[mask])
        m["critic/vf_explained_var"] = (1.0 - torch.var(ret[mask] - vals[mask]) / (var_ret + 1e-5)).item()
    m.update({f"response_length/{k.split('/')[-1]}": v for k, v in _stats("x", resp_len).items()})
    m["response_length/clip_ratio"] = (resp_len == R).float().mean().item()
    if nz.any():
        m.update({f"response_length_non_aborted/{k.split('/')[-1]}": v for k, v in _stats("x", resp_len[nz]).items()})
        m["response_length_non_aborted/clip_ratio"] = (resp_len[nz] == R).float().mean().item()
    m["response/aborted_ratio"] = aborted.float().mean().item()
    m.update({f"prompt_length/{k.split('/')[-1]}": v for k, v in _stats("x", prompt_len).items()})
    m["prompt_length/clip_ratio"] = (prompt_len == P).float().mean().item()
    if "__num_turns__" in batch.non_tensor_batch:
        nt = np.asarray(batch.non_tensor_batch["__num_turns__"], dtype=np.float64)
        m.update({"num_turns/min": nt.min(), "num_turns/max": nt.max(), "num_turns/mean": nt.mean()})
    return m


def compute_timing_metrics(batch: DataProto, timing_raw: dict[str, float]) -> dict[str, Any]:
    info = _compute_response_info(batch)
    n_prompt = float(info["prompt_length"].sum())
    n_resp = float(info["response_length"].sum())
    tokens = {"gen": n_resp, **{k: n_prompt + n_resp for k in ("ref", "values", "adv", "update_critic", "update_actor",
                                                                "old_log_prob")}}
    out = {f"timing_s/{k}": v for k, v in timing_raw.items()}
    out.update({f"timing_per_token_ms/{k}": timing_raw[k] * 1000 / tokens[k] for k in set(tokens) & set(timing_raw)
                if tokens[k] > 0})
    return out


def compute_throughout_metrics(batch: DataProto, timing_raw: dict[str, float], n_gpus: int) -> dict[str, Any]:
    """``perf/throughput`` = tokens (prompt + response) per second per GPU over the whole step."""
    total = sum(batch.meta_info["global_token_num"])
    t = timing_raw["step"]
    return {"perf/total_num_tokens": total, "perf/time_per_step": t, "perf/throughput": total / (t * n_gpus)}


def compute_variance_proxy_metrics(batch: DataProto, gradient_norm: float | None = None) -> dict[str, float]:
    """Cheap proxies for the variance of the policy-gradient estimator (per-sequence advantage energy)."""
    out = {}
    if "advantages" in batch.batch.keys() and "response_mask" in batch.batch.keys():
        a, m = batch.batch["advantages"], batch.batch["response_mask"].float()
        seq = (a * m).sum(-1)
        out["variance_proxy/adv_seq_sq_mean"] = seq.pow(2).mean().item()
        out["variance_proxy/adv_token_sq_mean"] = VF.masked_mean(a.pow(2), m).item()
    if gradient_norm is not None:
        out["variance_proxy/grad_norm_sq"] = float(gradient_norm) ** 2
    return out


def bootstrap_metric(data: list, subset_size: int, reduce_fns: list[Callable], n_bootstrap: int = 1000, seed: int = 42):
    rng = np.random.RandomState(seed)
    vals = [[] for _ in reduce_fns]
    for _ in range(n_bootstrap):
        idx = rng.choice(len(data), size=subset_size, replace=True)
        sub = [data[i] for i in idx]
        for j, fn in enumerate(reduce_fns):
            vals[j].append(fn(sub))
    return [(float(np.mean(v)), float(np.std(v))) for v in vals]


def calc_maj_val(data: list[dict], vote_key: str, val_key: str) -> float:
    votes = defaultdict(list)
    for d in data:
        votes[d[vote_key]].append(d[val_key])
    return max(votes.values(), key=len)[0]


def process_validation_metrics(data_sources: list[str], sample_uids: list[str], infos_dict: dict[str, list],
                               seed: int = 42) -> dict[str, dict[str, dict[str, float]]]:
    """Group validation samples by data source and prompt; report mean@N, best/worst@k (bootstrap) and maj@k."""
    grouped: dict = defaultdict(lambda: defaultdict(lambda: defaultdict(list)))
    for i, (ds, uid) in enumerate(zip(data_sources, sample_uids)):
        for name, vals in infos_dict.items():
            grouped[ds][uid][name].append(vals[i])
    per_prompt: dict = defaultdict(lambda: defaultdict(lambda: defaultdict(list)))
    for ds, by_uid in grouped.items():
        for uid, by_var in by_uid.items():
            for var, vals in by_var.items():
                if not vals or isinstance(vals[0], str) or var == "pred":
                    continue
                n = len(vals)
                per_prompt[ds][var][f"mean@{n}"].append(float(np.mean(vals)))
                if n > 1:
                    per_prompt[ds][var][f"std@{n}"].append(float(np.std(vals)))
                    ks = sorted({k for k in [2, 4, 8, 16, 32, 64] if k < n} | {n})
                    for k in ks:
                        (bm, _), (wm, _) = bootstrap_metric(vals, k, [np.max, np.min], n_bootstrap=200, seed=seed)
                        per_prompt[ds][var][f"best@{k}/mean"].append(bm)
                        per_prompt[ds][var][f"worst@{k}/mean"].append(wm)
                        if "pred" in by_var:
                            pairs = [{"val": v, "pred": p} for v, p in zip(vals, by_var["pred"])]
                            (mm, _), = bootstrap_metric(pairs, k, [partial(calc_maj_val, vote_key="pred", val_key="val")],
                                                        n_bootstrap=200, seed=seed)
                            per_prompt[ds][var][f"maj@{k}/mean"].append(mm)
    return {ds: {var: {m: float(np.mean(v)) for m, v in ms.items()} for var, ms in by_var.items()}
            for ds, by_var in per_prompt.items()}
