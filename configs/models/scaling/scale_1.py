"""Smallest model of the scaling series with the vocabulary size left open: instantiate with
`instantiate(conf.model, _tags_={"n_vocab": ...})`."""

from halite_b200.conf import call, field, tag

from .base import transformer

conf = field(model=call[transformer](tag("n_vocab"), 96, 4, 24, 3, call[int](96 * 3.5), 2048,
                                     rms_norm_epsilon=1e-6, post_norm=True))
