"""``ZirivikConfig``: the Zirivik decoder's config.json.

The class is the Python name of the host's ``ZirivikConfig`` (``csrc/host/config_zirivik.cpp``): keys ``architecture``
("Zirivik"), ``vocab``, ``width``, ``embedding.scale``, ``norm.eps``, ``logit_softcap`` and ``layers`` - a list whose
entries name a mixer (``type`` "retention" or "attention", sizes and constants under ``mixer``) and a feed-forward
(``mlp``: dense, a mixture of experts, or null) each, so the order and mix of layers is the file's.
"""
from __future__ import annotations

from .base import ModelConfig


class ZirivikConfig(ModelConfig):
    @classmethod
    def from_dict(cls, d: dict) -> "ZirivikConfig":
        d = dict(d)
        d.setdefault("architecture", "Zirivik")
        return super().from_dict(d)
