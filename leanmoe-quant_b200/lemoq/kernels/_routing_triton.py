"""Compatibility name: the reference exposes the routing op as
``lemoq.kernels._routing_triton.routing_softmax_topk`` (src/lemoq/kernels/_routing_triton.py:88).
The implementation here is the CUDA kernel of :mod:`lemoq.kernels.routing`; no Triton is involved."""

from lemoq.kernels.routing import routing_softmax_topk  # noqa: F401

__all__ = ["routing_softmax_topk"]
