"""Minerva-style 4-shot MATH (algebra subset by default): greedy decoding, stop at the next
"Problem:"."""

from functools import partial

from halite_b200.conf import field, function
from halite_b200.data.preprocess import Map, SelectFeatures
from halite_b200.projects.common.template import get_render_fn
from halite_b200.projects.eval.dataset import first_n, hf_dataset

from .eval import evaluate, fewshot_samples, record_to_input

fewshot_template = """{% for shot in fewshot %}
Problem:
{{ shot.problem }}

Solution: {{ shot.solution }}

{% endfor %}"""


def subject_task(subject):
    return field(
        name=f"minerva_math_{subject}",
        dataset=hf_dataset("EleutherAI/hendrycks_math", subject, split="test"),
        evaluate_fn=function(evaluate),
        preprocess=[SelectFeatures(keys=("problem", "solution")), Map(function(record_to_input))],
        sampling_params=field(max_new_tokens=512, top_k=1, stop=["Problem:"]),
        fewshot=field(sampler=partial(first_n, n=4), samples=function(fewshot_samples)),
        prefix=get_render_fn(template=fewshot_template),
    )


task = subject_task("algebra")
conf = field(tasks=[task])
