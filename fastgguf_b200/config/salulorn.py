"""``SalulornConfig``: the Salulorn decoder's config.json.

The class is the Python name of the host's ``SalulornConfig`` (``csrc/host/config_salulorn.cpp``): keys ``architecture``
("Salulorn"), ``vocab``, ``width``, ``norm.eps``, ``layers`` - a list whose entries name a mixer (``type`` "gla",
"attention" or "latent_attention", sizes and constants under ``mixer``) and a dense feed-forward (``mlp``, or null) - and
an optional ``loop`` (``start``, ``stop``, ``times``): a span of layers that runs several times in a row.
"""
from __future__ import annotations

from .base import ModelConfig


class SalulornConfig(ModelConfig):
    @classmethod
    def from_dict(cls, d: dict) -> "SalulornConfig":
        d = dict(d)
        d.setdefault("architecture", "Salulorn")
        return super().from_dict(d)
