"""Offline scoring of a file of generations: a parquet (or jsonl) table with, per row, N responses, the data source
and the reward-model record holding the ground truth. Prints and returns ``test_score/<data_source>`` means.

Rows are scored in a process pool (rule rewards are CPU-bound python). Parity target: ``verl/trainer/main_eval.py:35-83``.
"""

from __future__ import annotations

import concurrent.futures as cf
import os
import sys
from collections import defaultdict
from typing import Optional, Sequence

import numpy as np

from ..utils.config import load_config

CONFIG_DIR = os.path.join(os.path.dirname(__file__), "config")


def _score_row(args):
    fn_path, fn_name, data_source, responses, reward_data = args
    if fn_path:
        from .ppo.reward import load_extern_object

        fn = load_extern_object(fn_path, fn_name)
    else:
        from ..utils.reward_score import default_compute_score as fn
    gt = reward_data["ground_truth"] if isinstance(reward_data, dict) else reward_data
    scores = []
    for r in list(responses):
        s = fn(data_source, r, gt)
        scores.append(float(s["score"]) if isinstance(s, dict) else float(s))
    return data_source, float(np.mean(scores)) if scores else 0.0


def _read_table(path: str):
    import pandas as pd

    path = os.path.expanduser(path)
    return pd.read_json(path, lines=True) if path.endswith((".jsonl", ".json")) else pd.read_parquet(path)


def evaluate(config) -> dict:
    df = _read_table(config.data.path)
    crf = config.get("custom_reward_function") or {}
    jobs = [(crf.get("path"), crf.get("name", "compute_score"), df[config.data.data_source_key][i], df[config.data.response_key][i],
             df[config.data.reward_model_key][i]) for i in range(len(df))]
    per_source = defaultdict(list)
    workers = int(config.get("num_workers", 1) or 1)
    if workers > 1 and len(jobs) > 1:
        with cf.ProcessPoolExecutor(max_workers=workers) as ex:
            results = list(ex.map(_score_row, jobs, chunksize=max(1, len(jobs) // (4 * workers))))
    else:
        results = [_score_row(j) for j in jobs]
    for src, s in results:
        per_source[src].append(s)
    return {f"test_score/{k}": float(np.mean(v)) for k, v in per_source.items()}


def main(argv: Optional[Sequence[str]] = None):
    argv = list(sys.argv[1:] if argv is None else argv)
    metrics = evaluate(load_config(CONFIG_DIR, "evaluation", argv))
    print(metrics)
    return metrics


if __name__ == "__main__":
    main()
