"""Scores for the synthetic token-id tasks when they are evaluated through the text path: the response string is
a space-separated list of token ids and the ground truth is the target residue modulo 7."""


def compute_score(solution_str: str, ground_truth, extra_info=None) -> float:
    toks = [int(t) for t in solution_str.split() if t.lstrip("-").isdigit()]
    if not toks:
        return 0.0
    mod = int((extra_info or {}).get("modulus", 7)) if isinstance(extra_info, dict) else 7
    return sum(1 for t in toks if t % mod == int(ground_truth) % mod) / len(toks)
