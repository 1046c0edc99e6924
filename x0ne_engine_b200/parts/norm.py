"""RMSNorm with the residual add fused in front of it."""
from __future__ import annotations

from typing import List, Mapping

import torch

from ..config.spec import PartSpec
from ..csrc import ops
from ..weights.loader import TensorNeed
from .base import NORMS, Norm


class PostNormed:
    """A sublayer's result that is still to be normed by `norm` (an RMSNorm of its own) before it joins the
    residual: what a layer with norms after its sublayers hands to the next add.  The norm that takes it
    norms the delta in float32, adds it, and norms the sum, in one launch."""
    __slots__ = ("delta", "norm")

    def __init__(self, delta: torch.Tensor, norm: "RMSNorm"):
        self.delta = delta
        self.norm = norm


class RMSNorm(Norm):
    """out = r * rsqrt(mean(r^2) + eps) * w with r = resid + delta, in float32; eps inside the
    root, the weight multiplies directly (x0ne-core/kernels/cuda/rmsnorm.cu:11-20).
    Parameters: size, eps, names.weight."""
    replayable = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.size = int(spec["size"])
        self.eps = float(spec["eps"])
        self.weight = None

    @staticmethod
    def tensor_needs(spec: PartSpec) -> List[TensorNeed]:
        return [TensorNeed(spec["names"]["weight"], (int(spec["size"]),), role="vector", init="norm")]

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.weight = tensors[self.spec["names"]["weight"]]

    def add_norm(self, ctx, resid, delta, out, n_rows, rows=None):
        if isinstance(delta, PostNormed):
            ops.add_normed_rmsnorm(resid, delta.delta, delta.norm.weight, delta.norm.eps, self.weight, out, n_rows, self.eps, rows)
        else:
            ops.add_rmsnorm(resid, delta, self.weight, out, n_rows, self.eps, rows)


NORMS.register("rmsnorm", RMSNorm)
