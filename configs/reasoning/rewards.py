"""Reward functions for reasoning RL: answer correctness inside <answer>...</answer> and the
think/answer format check (reference: configs/reasoning/rewards.py:6-93)."""

import re

import torch

_ANSWER = re.compile(r"<answer>(.*)</answer>", re.DOTALL)
_FORMAT = re.compile(r".*</think>.*<answer>.*</answer>.*", re.DOTALL)


def get_answer(text: str) -> str:
    m = _ANSWER.search(text)
    return m.group(1) if m else "None"


class MathVerify:
    def __init__(self, timeout_score=0, multiprocess_mode=False, timeout_seconds=5):
        from halite_b200.projects.rewards.math_verify import math_metric, timeout

        self.timeout_score = timeout_score
        targets = {}
        try:
            from math_verify.parser import ExprExtractionConfig, LatexExtractionConfig

            targets = dict(gold_extraction_target=(LatexExtractionConfig(),),
                           pred_extraction_target=(ExprExtractionConfig(), LatexExtractionConfig()))
        except ImportError:
            pass
        fn = math_metric(**targets)
        self.verify_fn = timeout(timeout_seconds)(fn) if multiprocess_mode else fn

    def verify(self, model_output, ground_truth):
        from halite_b200.projects.rewards.math_verify import TimeoutException

        answer = get_answer(model_output)
        if answer == "None":
            return 0.0
        try:
            score, _ = self.verify_fn([ground_truth], ["\\boxed{" + answer + "}"])
            return float(score)
        except TimeoutException:
            return float(self.timeout_score)
        except Exception:  # noqa: BLE001  (unparseable gold or prediction)
            return 0.0

    def __call__(self, model_output, ground_truth):
        return torch.tensor([self.verify(o, t) for o, t in zip(model_output, ground_truth)], dtype=torch.float32)


class FormatReward:
    def check_format(self, model_output):
        return 1.0 if _FORMAT.fullmatch(model_output) else 0.0

    def __call__(self, model_output):
        return torch.tensor([self.check_format(o) for o in model_output], dtype=torch.float32)
