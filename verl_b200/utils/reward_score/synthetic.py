"""Synthetic rule reward of the benchmark configurations: 1.0 iff (last response token id mod 7) equals
(sum of prompt token ids mod 7). Works on token ids, so no tokenizer is involved."""


def compute_score_from_ids(prompt_ids, response_ids) -> float:
    if len(response_ids) == 0:
        return 0.0
    return 1.0 if int(response_ids[-1]) % 7 == int(sum(int(t) for t in prompt_ids)) % 7 else 0.0


def compute_score_from_text(solution_str: str, ground_truth) -> float:
    toks = solution_str.split()
    try:
        return 1.0 if toks and int(toks[-1]) % 7 == int(ground_truth) % 7 else 0.0
    except ValueError:
        return 0.0
