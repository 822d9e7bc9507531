"""A CPU stand-in for the operator, for host-side tests of code that calls it (the UNet harness).

Test infrastructure only: it computes Linear in FP32 with torch on the CPU and rounds to FP16 where
the operator does. Nothing in the package imports it; the product path has no CPU fallback."""
from __future__ import annotations

import torch
import torch.nn.functional as F


class FakeWeight:
    def __init__(self, values: torch.Tensor):
        self.values = values.to(torch.float16)
        self.n, self.k = values.shape


class _FakeContext:
    device = 0

    def set_stream(self, stream):
        pass


class _FakePlan:
    def __init__(self, ops, calls):
        self.ops, self.calls = ops, list(calls)
        for call in self.calls:
            m = call.x.numel() // call.weight.k
            call.y = torch.empty(tuple(call.x.shape[:-1]) + (call.weight.n,), dtype=torch.float16)
        self.runs = 0

    def run(self):
        self.runs += 1
        for call in self.calls:
            call.y.copy_(self.ops._compute(call.x, call.weight, call.bias, call.activation, None))
        return [call.y for call in self.calls]

    def close(self):
        pass


class FakeOps:
    """Same call surface as the package's Ops for the methods the harness uses; records every call."""

    def __init__(self):
        self.ctx = _FakeContext()
        self.log = []          # (kind, rows, n, k, has_bias, activation, has_residual)

    @staticmethod
    def fp16_weight(values):
        return FakeWeight(values)

    def _compute(self, x, weight, bias, activation, residual):
        y = F.linear(x.float(), weight.values.float()).to(torch.float16)       # projection rounded to FP16
        if activation == 0:
            if bias is not None:
                y = (y.float() + bias.float()).to(torch.float16)               # __hadd
            if residual is not None:
                y = (y.float() + residual.float()).to(torch.float16)
            return y
        z = y.float() + bias.float()
        if activation == 1:
            return F.silu(z).to(torch.float16)
        if activation == 4:
            value, gate = z.chunk(2, dim=-1)
            return (value * F.gelu(gate)).to(torch.float16)
        raise NotImplementedError(activation)

    def layer_norm(self, x, gamma, beta, epsilon=1.0e-5, out=None):
        self.log.append(("layer_norm", x.numel() // x.shape[-1], x.shape[-1], 0, True, 0, False))
        return F.layer_norm(x.float(), (x.shape[-1],), gamma.float(), beta.float(), epsilon).to(torch.float16)

    def group_norm_nhwc(self, x, gamma, beta, groups, epsilon=1.0e-5, silu=False, channel_bias=None):
        self.log.append(("group_norm", x.shape[0], x.shape[1], 0, True, int(silu), channel_bias is not None))
        if channel_bias is not None:
            x = (x.float() + channel_bias.float()[:, :, None, None]).to(torch.float16)
        y = F.group_norm(x.float(), groups, gamma.float(), beta.float(), epsilon)
        if silu:
            y = F.silu(y)
        return y.to(torch.float16).contiguous(memory_format=torch.channels_last)

    def bias_residual_add_nhwc(self, x, bias, residual):
        biased = (x.float() + bias.float()[None, :, None, None]).to(torch.float16)
        return (biased.float() + residual.float()).to(torch.float16).contiguous(memory_format=torch.channels_last)

    def linear(self, x, weight, bias=None, *, residual=None, out=None, **_):
        self.log.append(("linear", x.numel() // weight.k, weight.n, weight.k, bias is not None, 0, residual is not None))
        y = self._compute(x, weight, bias, 0, residual)
        if out is not None:
            out.copy_(y)
            return out
        return y

    def linear_activation(self, x, weight, bias, activation, **_):
        self.log.append(("linear_activation", x.numel() // weight.k, weight.n, weight.k, True, int(activation), False))
        return self._compute(x, weight, bias, int(activation), None)

    def linear_grouped(self, calls):
        out = []
        for call in calls:
            self.log.append(("grouped", call.x.numel() // call.weight.k, call.weight.n, call.weight.k, call.bias is not None,
                             int(call.activation), False))
            out.append(self._compute(call.x, call.weight, call.bias, int(call.activation), None))
        return out

    def plan(self, calls):
        calls = list(calls)
        for call in calls:
            self.log.append(("plan", call.x.numel() // call.weight.k, call.weight.n, call.weight.k, call.bias is not None,
                             int(call.activation), False))
        return _FakePlan(self, calls)
