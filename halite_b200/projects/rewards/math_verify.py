"""Answer checking for math RL rewards (reference: projects/rewards/math_verify.py:12-147).

`math_metric` builds a sample-level function `(golds, predictions) -> (score, strings)` that
extracts expressions with the `math_verify` package and scores 1.0 when any prediction matches
any gold. `timeout` runs a function in a forked child and raises when it overruns, so a
pathological sympy simplification cannot stall a training step. Without `math_verify`
installed a small sympy / string comparison stands in.
"""

from __future__ import annotations

import functools
import multiprocessing as mp
import queue
import re
from typing import Callable, Sequence

try:
    from math_verify.errors import TimeoutException
except ImportError:  # pragma: no cover
    class TimeoutException(Exception):
        pass


def _fallback_equal(gold: str, pred: str, precision: int) -> bool:
    """String match after stripping TeX wrappers, then numeric / symbolic equality via sympy."""
    def clean(s):
        s = s.strip().strip("$")
        m = re.search(r"\\boxed\{(.*)\}", s, re.DOTALL)
        if m:
            s = m.group(1)
        s = re.sub(r"\\left|\\right|\\!|\\,|\;|\s+", "", s)
        s = re.sub(r"\\d?frac\{([^{}]*)\}\{([^{}]*)\}", r"(\1)/(\2)", s)
        return s

    g, p = clean(gold), clean(pred)
    if g == p:
        return True
    try:
        import sympy

        eg, ep = sympy.sympify(g.replace("^", "**")), sympy.sympify(p.replace("^", "**"))
        if eg.is_number and ep.is_number:
            return abs(float(eg) - float(ep)) <= 10.0 ** -precision
        return sympy.simplify(eg - ep) == 0
    except Exception:  # noqa: BLE001
        return False


def math_metric(gold_extraction_target: Sequence | None = None, pred_extraction_target: Sequence | None = None,
                aggregation_function: Callable[[list[float]], float] = max, precision: int = 6):
    try:
        from math_verify import grader, parser
        from math_verify.grader import verify
        from math_verify.parser import ExprExtractionConfig, parse
    except ImportError:
        def sample_level_fn(golds, predictions):
            scores = [1.0 if any(_fallback_equal(g, p, precision) for g in golds) else 0.0 for p in predictions]
            return aggregation_function(scores), (list(golds), list(predictions))

        return sample_level_fn

    gold_t = tuple(gold_extraction_target or (ExprExtractionConfig(),))
    pred_t = tuple(pred_extraction_target or (ExprExtractionConfig(),))

    def sample_level_fn(golds, predictions):
        # the package's own signal-based timeouts do not work off the main thread: disable them
        grader.TIMEOUT_WARNING_SHOWN = True
        parser.TIMEOUT_WARNING_SHOWN = True
        preds = [parse(p, pred_t, parsing_timeout=None) for p in predictions]
        gold = [parse(g, gold_t, parsing_timeout=None) for g in golds]
        if any(len(g) == 0 for g in gold):
            raise ValueError(f"no gold target could be extracted: {golds}")
        scores = [1.0 if any(verify(g, p, precision, timeout_seconds=None) for g in gold) else 0.0 for p in preds]
        strings = ([str(x) for g in gold for x in g], [str(x) for p in preds for x in p])
        return aggregation_function(scores), strings

    return sample_level_fn


def timeout(timeout_seconds: float):
    """Decorator: run the call in a forked child; TimeoutException if it takes too long."""
    ctx = mp.get_context("fork")

    def decorator(fn):
        @functools.wraps(fn)
        def wrapper(*args, **kwargs):
            q = ctx.Queue()

            def child():
                try:
                    q.put((True, fn(*args, **kwargs)))
                except Exception as e:  # noqa: BLE001
                    q.put((False, e))

            proc = ctx.Process(target=child)
            proc.start()
            try:
                ok, value = q.get(timeout=timeout_seconds)
            except queue.Empty:
                proc.terminate()
                proc.join()
                raise TimeoutException(f"{fn.__name__} did not finish within {timeout_seconds} s") from None
            proc.join()
            if not ok:
                raise value
            return value

        return wrapper

    return decorator
