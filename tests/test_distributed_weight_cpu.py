"""A weight sharded by the caller: the module assembles it for the GEMMs through the distributed-weight
protocol and hands the full gradient back (reference contract: ``pytorch/distributed_weight.py``)."""
import torch

import transformerengine_b200 as te
from transformerengine_b200 import distributed_weight as DW


class ShardedWeight(torch.nn.Parameter):
    """Holds the first half of the rows; the second half lives 'elsewhere' (here: an attribute)."""
    is_distributed_weight = True

    def materialize_group_for_forward(self):
        self.calls["fwd"] += 1
        return torch.cat([self.detach(), self.other_shard], dim=0)

    def materialize_group_for_backward(self):
        self.calls["bwd"] += 1
        return torch.cat([self.detach(), self.other_shard], dim=0)

    def finalize_group_grads(self, wgrad):
        # "reduce-scatter": keep the rows of this shard, remember the rest for the test
        self.calls["grads"] += 1
        self.full_grad = wgrad.detach().clone()
        return wgrad[: self.shape[0]].to(self.dtype)

    def grad_buffer(self):
        return self.grad


def test_dispatch_helpers_pass_plain_tensors_through():
    w = torch.randn(4, 4)
    assert not DW.is_distributed_weight(w)
    assert DW.materialize_weight_for_forward(w)[0] is w
    assert DW.finalize_weight_grads([w], [w])[0] is w


def test_linear_runs_on_a_sharded_weight():
    torch.manual_seed(0)
    lin = te.Linear(32, 64, bias=True, params_dtype=torch.float32, device="cpu")
    full = lin.weight.detach().clone()
    shard = ShardedWeight(full[:32].clone())
    shard.other_shard = full[32:].clone()
    shard.calls = {"fwd": 0, "bwd": 0, "grads": 0}
    del lin._parameters["weight"]
    lin.register_parameter("weight", shard)
    x = torch.randn(16, 32, requires_grad=True)
    y = lin(x)
    ref = torch.nn.functional.linear(x, full, lin.bias)
    torch.testing.assert_close(y, ref, rtol=1e-5, atol=1e-5)
    y.sum().backward()
    assert shard.calls == {"fwd": 1, "bwd": 1, "grads": 1}
    gref = torch.ones(16, 64).t() @ x.detach()
    torch.testing.assert_close(shard.full_grad.float(), gref, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(shard.grad, gref[:32], rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(x.grad, torch.ones(16, 64) @ full, rtol=1e-4, atol=1e-4)
    # quantized autocast goes through the same hooks
    with te.autocast(enabled=True, recipe=te.recipe.MXFP8BlockScaling()):
        yq = lin(x)
    assert (yq - ref).abs().max() < 0.1 * ref.abs().max()
