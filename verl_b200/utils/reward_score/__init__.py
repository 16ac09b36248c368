"""Rule-based scorers selected by ``data_source`` (reference: ``verl/utils/reward_score/__init__.py:19``)."""

from __future__ import annotations

from . import geo3k, gsm8k, math_dapo, math_reward, math_verify, prime_code, prime_math, rlla, sandbox_fusion, search_r1_like_qa_em, synthetic

__all__ = ["default_compute_score"]


def default_compute_score(data_source: str, solution_str: str, ground_truth, extra_info=None, **kwargs):
    if data_source in ("openai/gsm8k", "gsm8k"):
        return gsm8k.compute_score(solution_str, ground_truth)
    if data_source in ("lighteval/MATH", "DigitalLearningGmbH/MATH-lighteval", "HuggingFaceH4/MATH-500", "math"):
        return math_reward.compute_score(solution_str, ground_truth)
    if data_source in ("math_dapo", "math", "math_dapo_reasoning") or str(data_source).startswith("aime"):
        return math_dapo.compute_score(solution_str, ground_truth)
    if data_source in ("numina_aops_forum", "numina_synthetic_math", "numina_amc_aime", "numina_synthetic_amc", "numina_cn_k12", "numina_olympiads"):
        return float(prime_math.compute_score(solution_str, ground_truth)[0])
    if data_source in ("codecontests", "apps", "codeforces", "taco"):
        url = kwargs.get("sandbox_fusion_url")
        if url:        # a remote sandbox service is configured: post the test cases there
            return float(sandbox_fusion.compute_score(url, kwargs.get("concurrent_semaphore"), int(kwargs.get("memory_limit_mb", 1024)),
                                                      solution_str, ground_truth, continuous=True)[0])
        # otherwise the test cases run in a local subprocess sandbox
        return float(prime_code.compute_score(solution_str, ground_truth, continuous=True)[0])
    if data_source in ("hiyouga/geometry3k", "geo3k"):
        return geo3k.compute_score(solution_str, ground_truth)
    if data_source in ("searchR1_nq", "searchR1_triviaqa", "searchR1_popqa", "searchR1_hotpotqa", "searchR1_2wikimultihopqa",
                       "searchR1_musique", "searchR1_bamboogle"):
        return search_r1_like_qa_em.compute_score(solution_str, ground_truth)
    if data_source in ("rlla", "rlla_gdpo", "toolrl"):
        return rlla.compute_score(data_source, solution_str, ground_truth, extra_info or {})
    if data_source in ("math_verify",) or (kwargs.get("use_math_verify") and math_verify.available()):
        return math_verify.compute_score(solution_str, ground_truth)
    if data_source in ("synthetic/mod7", "mod7"):
        return synthetic.compute_score_from_text(solution_str, ground_truth)
    raise NotImplementedError(f"Reward function is not implemented for data_source={data_source!r}")
