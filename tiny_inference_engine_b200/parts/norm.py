"""RMSNorm: (x * 1/sqrt(mean(x^2) + eps)) * w, sums and scale in float32
(src/backend/cpu/cpu_backend.cpp:141-159). The weight is kept in float32 whatever the
checkpoint stores (src/model/qwen3.cpp:60-71)."""
from __future__ import annotations

import torch

from .. import ops
from ..weights.loader import TensorNeed
from .base import Norm, register_part


class RMSNorm(Norm):
    launches_only = True
    takes_split_sum = True      # add_norm adds the partial sums of a split product itself
    fusable_rms = True          # exactly the formula above, with `weight` (float32) and `eps`

    def __init__(self, spec, dtype, prefix: str = ""):
        self.name = prefix + spec["name"]
        self.size = int(spec["size"])
        self.eps = float(spec["eps"])
        self.dtype = dtype
        self.weight = None

    def needs(self):
        return {self.name: TensorNeed((self.size,), "norm")}

    def bind(self, get):
        self.weight = get(self.name).to(torch.float32).contiguous()

    def add_norm(self, x, delta, out, rows=None):
        if isinstance(delta, ops.NormedDelta):      # a sublayer's output that passes a norm of its own on its way in
            ops.add_normed_rmsnorm(x, delta, self.weight, self.eps, out, rows)
        else:
            ops.add_rmsnorm(x, delta, self.weight, self.eps, out, rows)

    def rows(self, x, out):
        ops.rmsnorm_rows(x, self.weight, self.eps, out)


register_part("norm", "rmsnorm", RMSNorm, replace=True)


class RMSNormOnePlus(RMSNorm):
    """RMSNorm whose weight is stored as its distance from one: (x / sqrt(mean(x^2) + eps)) * (1 + w). The sum
    1 + w is formed once, in float32, when the weight is bound; after that it is the formula of `RMSNorm`."""

    def bind(self, get):
        self.weight = (get(self.name).to(torch.float32) + 1.0).contiguous()


register_part("norm", "rmsnorm_one_plus", RMSNormOnePlus, replace=True)


class GroupedRMSNorm(Norm):
    """RMS norm in groups: a row is split into `groups` equal consecutive parts, each divided by its own
    sqrt(mean(part^2) + eps), and the whole multiplied by the weight. With one group it is `RMSNorm`'s formula, through
    the kernel that also serves layers whose sublayers read one stream side by side (`parallel_taps`)."""
    launches_only = True
    takes_split_sum = True

    def __init__(self, spec, dtype, prefix: str = ""):
        self.name = prefix + spec["name"]
        self.size = int(spec["size"])
        self.eps = float(spec["eps"])
        self.groups = int(spec.params.get("groups", 1))
        if self.groups <= 0 or self.size % self.groups:
            from ..errors import InvalidArgument
            raise InvalidArgument(f"a norm over {self.size} columns cannot have {self.groups} equal groups")
        self.dtype = dtype
        self.weight = None

    def needs(self):
        return {self.name: TensorNeed((self.size,), "norm")}

    def bind(self, get):
        self.weight = get(self.name).to(torch.float32).contiguous()

    def add_norm(self, x, delta, out, rows=None):
        if isinstance(delta, ops.NormedDelta):
            raise NotImplementedError("a grouped norm takes a plain delta or partial sums, not one that still has a norm to pass")
        ops.group_norm_taps(x, self.groups, self.eps, self.weight, out, delta=delta, rows=rows)

    def rows(self, x, out):
        if x.dtype != torch.float32 or not x.is_contiguous():
            raise NotImplementedError("a grouped norm over other views than contiguous float32 rows")
        ops.group_norm_taps(x, self.groups, self.eps, self.weight, out)


register_part("norm", "grouped_rmsnorm", GroupedRMSNorm, replace=True)


class DynamicTanh(Norm):
    """A norm without statistics: tanh(alpha * x) * weight + bias, element by element, with a learned scalar alpha
    (`<name>.alpha`) and a bias vector (`<name>.b`) stored beside the weight. No mean, no variance, no eps. The residual
    add ahead of it is fused in as for the other norms, and it adds sums of sublayer outputs with factors (`ops.ScaledSum`)
    and the partial sums of split products itself, in float32."""
    launches_only = False
    takes_split_sum = True
    takes_scaled_sum = True

    def __init__(self, spec, dtype, prefix: str = ""):
        self.name = prefix + spec["name"]
        self.size = int(spec["size"])
        self.dtype = dtype
        self.weight = self.bias = None
        self.alpha = 1.0

    def needs(self):
        return {self.name: TensorNeed((self.size,), "norm"), self.name + ".b": TensorNeed((self.size,), "norm"),
                self.name + ".alpha": TensorNeed((), "norm")}

    def bind(self, get):
        self.weight = get(self.name).to(torch.float32).contiguous()
        self.bias = get(self.name + ".b").to(torch.float32).contiguous()
        self.alpha = float(get(self.name + ".alpha").to(torch.float32).reshape(-1)[0].item())

    def add_norm(self, x, delta, out, rows=None):
        if isinstance(delta, ops.NormedDelta):
            raise NotImplementedError("a dynamic tanh takes a plain delta, partial sums or a scaled sum, not one that still has a norm to pass")
        ops.add_tanh_norm(x, delta, self.alpha, self.weight, self.bias, out, rows)

    def rows(self, x, out):
        if x.dtype != torch.float32 or not x.is_contiguous():
            raise NotImplementedError("a dynamic tanh over other views than contiguous float32 rows")
        ops.add_tanh_norm(x, None, self.alpha, self.weight, self.bias, out)


register_part("norm", "dynamic_tanh", DynamicTanh, replace=True)
