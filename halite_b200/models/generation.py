"""Dense-cache generation loop with logits processors
(reference: transformers/generation.py:5-384). The production sampling path is the paged engine
in `halite_b200.infer`; this mixin is the small self-contained loop used for sanity checks,
conversion tests and models the engine does not cover.

All sequences stay in the batch until every one has finished (finished rows are fed the pad
token and their outputs ignored), so shapes are static and the loop never re-slices caches.
"""

from __future__ import annotations

import torch
import torch.distributed as dist


class LogitsProcessor:
    def __call__(self, input_ids, scores):
        raise NotImplementedError


class LogitsProcessorList(list):
    def __call__(self, input_ids, scores, **kwargs):
        for p in self:
            scores = p(input_ids, scores)
        return scores


class StoppingCriteriaList(list):
    def __call__(self, input_ids, scores):
        return any(c(input_ids, scores) for c in self)


class MaxLengthCriteria:
    def __init__(self, max_length):
        self.max_length = max_length

    def __call__(self, input_ids, scores):
        return input_ids.shape[-1] >= self.max_length


class TemperatureLogitsProcessor(LogitsProcessor):
    def __init__(self, temperature):
        if not temperature > 0:
            raise ValueError("temperature must be positive")
        self.temperature = temperature

    def __call__(self, input_ids, scores):
        return scores / self.temperature


class TopKLogitsProcessor(LogitsProcessor):
    def __init__(self, top_k, filter_value=-float("inf"), min_tokens_to_keep=1):
        self.top_k = max(int(top_k), min_tokens_to_keep)
        self.filter_value = filter_value

    def __call__(self, input_ids, scores):
        k = min(self.top_k, scores.shape[-1])
        kth = torch.topk(scores, k)[0][..., -1, None]
        return scores.masked_fill(scores < kth, self.filter_value)


class TopPLogitsProcessor(LogitsProcessor):
    def __init__(self, top_p, filter_value=-float("inf"), min_tokens_to_keep=1):
        if not 0 <= top_p <= 1:
            raise ValueError("top_p must be in [0, 1]")
        self.top_p, self.filter_value, self.min_keep = top_p, filter_value, min_tokens_to_keep

    def __call__(self, input_ids, scores):
        sorted_scores, order = torch.sort(scores, descending=True)
        cum = sorted_scores.softmax(-1).cumsum(-1)
        drop = cum - sorted_scores.softmax(-1) > self.top_p       # mass before the token already exceeds p
        drop[..., :self.min_keep] = False
        drop = drop.scatter(-1, order, drop)
        return scores.masked_fill(drop, self.filter_value)


class RepetitionPenaltyLogitsProcessor(LogitsProcessor):
    def __init__(self, penalty):
        if not penalty > 0:
            raise ValueError("penalty must be positive")
        self.penalty = penalty

    def __call__(self, input_ids, scores):
        seen = scores.gather(1, input_ids)
        seen = torch.where(seen < 0, seen * self.penalty, seen / self.penalty)
        return scores.scatter(1, input_ids, seen)


def _cached_length(cache):
    if not cache:
        return 0
    first = cache[0]
    if first is None:
        return 0
    return first.length if hasattr(first, "length") else first[0].shape[1]


class GenerationMixin:
    def get_logits_processor(self, temperature=1, top_k=0, top_p=1, repetition_penalty=1):
        procs = LogitsProcessorList()
        if repetition_penalty != 1:
            procs.append(RepetitionPenaltyLogitsProcessor(repetition_penalty))
        if temperature not in (0, 1):
            procs.append(TemperatureLogitsProcessor(temperature))
        if top_k > 0:
            procs.append(TopKLogitsProcessor(top_k))
        if top_p < 1:
            procs.append(TopPLogitsProcessor(top_p))
        return procs

    def get_stopping_criteria(self, max_length=None):
        crit = StoppingCriteriaList()
        if max_length is not None:
            crit.append(MaxLengthCriteria(max_length))
        return crit

    def prepare_inputs(self, input_ids=None, attention_mask=None, bos_token_id=None, device="cpu"):
        if input_ids is not None:
            return input_ids, attention_mask
        ids = torch.full((1, 1), bos_token_id, dtype=torch.int64, device=device)
        return ids, torch.ones_like(ids)

    def expand_inputs(self, input_ids=None, model_kwargs=None, expand_factor=1):
        if input_ids is not None:
            input_ids = input_ids.repeat_interleave(expand_factor, 0)
        kw = {k: (v.repeat_interleave(expand_factor, 0) if isinstance(v, torch.Tensor) else v)
              for k, v in (model_kwargs or {}).items()}
        return input_ids, kw

    def prepare_inputs_for_generation(self, input_ids, cache=None, attention_mask=None, use_cache=True, **kw):
        """First step feeds the whole prompt, later steps only the newest token."""
        if use_cache and _cached_length(cache) > 0:
            input_ids = input_ids[:, -1:]
        out = {"input_ids": input_ids, "cache": cache, "use_cache": use_cache}
        if attention_mask is not None and not bool(attention_mask.all()):
            out["attention_mask"] = attention_mask
        return out

    def update_model_kwargs_for_generation(self, outs, model_kwargs):
        if getattr(outs, "cache", None):
            model_kwargs["cache"] = outs.cache
        mask = model_kwargs.get("attention_mask")
        if mask is not None:
            model_kwargs["attention_mask"] = torch.cat((mask, mask.new_ones(mask.shape[0], 1)), -1)
        return model_kwargs

    @torch.no_grad()
    def generate(self, input_ids=None, mode="sample", max_length=None, max_new_tokens=None, bos_token_id=None,
                 eos_token_id=None, pad_token_id=None, temperature=1, top_k=0, top_p=1, repetition_penalty=1,
                 use_cache=True, synced_gpus=False, num_return_sequences=1, device="cpu", streamer=None,
                 generator=None, **kwargs):
        if input_ids is not None:
            if input_ids.ndim < 2:
                input_ids = input_ids.unsqueeze(0)
            device = input_ids.device
        input_ids, attention_mask = self.prepare_inputs(input_ids, kwargs.pop("attention_mask", None),
                                                        bos_token_id, device)
        model_kwargs = {"attention_mask": attention_mask, "use_cache": use_cache, **kwargs}
        if streamer is not None:
            streamer.put(input_ids.cpu())
        if max_new_tokens is not None:
            limit = input_ids.shape[1] + max_new_tokens
            max_length = limit if max_length is None else min(max_length, limit)
        if num_return_sequences > 1:
            input_ids, model_kwargs = self.expand_inputs(input_ids, model_kwargs, num_return_sequences)
        if mode != "sample":
            raise ValueError(f"unknown generation mode {mode!r}")
        return self.sample(input_ids, eos_token_id, pad_token_id, self.get_stopping_criteria(max_length),
                           self.get_logits_processor(temperature, top_k, top_p, repetition_penalty),
                           synced_gpus, streamer, greedy=temperature == 0, generator=generator, **model_kwargs)

    @torch.no_grad()
    def sample(self, input_ids, eos_token_id=None, pad_token_id=None, stopping_criteria=None,
               logits_processor=None, synced_gpus=False, streamer=None, greedy=False, generator=None,
               **model_kwargs):
        stopping_criteria = stopping_criteria or StoppingCriteriaList()
        logits_processor = logits_processor or LogitsProcessorList()
        eos = None
        if eos_token_id is not None:
            if pad_token_id is None:
                raise ValueError("if `eos_token_id` is defined, `pad_token_id` should be defined")
            eos = torch.as_tensor(eos_token_id, device=input_ids.device).view(-1)
        alive = torch.ones(input_ids.shape[0], dtype=torch.bool, device=input_ids.device)
        done_here = False
        while True:
            if synced_gpus:
                # ranks with nothing left keep stepping the model until every rank is finished
                flag = torch.tensor([0.0 if done_here else 1.0], device=input_ids.device)
                dist.all_reduce(flag)
                if flag.item() == 0:
                    break
            outs = self(**self.prepare_inputs_for_generation(input_ids, **model_kwargs))
            if synced_gpus and done_here:
                continue
            scores = logits_processor(input_ids, outs.logits[:, -1].float())
            if greedy:
                token = scores.argmax(-1)
            else:
                token = torch.multinomial(scores.softmax(-1), 1, generator=generator).squeeze(1)
            if eos is not None:
                token = torch.where(alive, token, torch.full_like(token, pad_token_id))
            input_ids = torch.cat((input_ids, token[:, None]), -1)
            if streamer is not None:
                streamer.put(token.cpu())
            model_kwargs = self.update_model_kwargs_for_generation(outs, model_kwargs)
            if eos is not None:
                alive = alive & ~(token[:, None] == eos[None, :]).any(-1)
                if not bool(alive.any()):
                    done_here = True
            if stopping_criteria(input_ids, None):
                done_here = True
            if done_here and not synced_gpus:
                break
        if streamer is not None:
            streamer.end()
        return input_ids
