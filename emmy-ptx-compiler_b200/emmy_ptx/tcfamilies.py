"""Tensor-core families (matmul, attention, fused MLP): pattern matching and template instantiation."""

from __future__ import annotations

from .families import Refusal


def match_matmul(src, strict: bool):
    raise Refusal("not built yet")


def match_attention(src, strict: bool):
    raise Refusal("not built yet")


def match_mlp(src, strict: bool):
    raise Refusal("not built yet")
