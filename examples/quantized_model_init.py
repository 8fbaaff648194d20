"""Parameters that live in FP8: ``te.quantized_model_init`` creates the weights quantized, the optimizer keeps the
fp32 master copy, and every step re-quantizes the weights from the master values.

    python examples/quantized_model_init.py --recipe mxfp8

What to look at: the module's ``weight`` is a ``QuantizedTensor`` (1 byte per element plus scales instead of 2 or 4);
``FusedAdam(master_weights=True)`` updates an fp32 master and writes the new values back quantized;
``preserve_high_precision_init_val`` keeps the unquantized initial values around so that the master weights start
from them and not from the rounded FP8 values; the state dict round trip keeps the payload bit-exact.
(Counterpart of the reference's ``examples/pytorch/quantized_model_init/main.py``.)
"""
import argparse
import io
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import transformerengine_b200 as te  # noqa: E402
from transformerengine_b200.common import recipe as R  # noqa: E402

RECIPES = {"delayed": R.DelayedScaling, "current": R.Float8CurrentScaling, "mxfp8": R.MXFP8BlockScaling}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--recipe", default="mxfp8", choices=sorted(RECIPES))
    ap.add_argument("--hidden", type=int, default=256)
    ap.add_argument("--steps", type=int, default=10)
    a = ap.parse_args(argv)
    cuda = torch.cuda.is_available()
    dev, dtype = ("cuda", torch.bfloat16) if cuda else ("cpu", torch.float32)
    recipe = RECIPES[a.recipe]()
    torch.manual_seed(0)
    with te.quantized_model_init(enabled=True, recipe=recipe, preserve_high_precision_init_val=True):
        mlp = te.LayerNormMLP(a.hidden, 4 * a.hidden, normalization="RMSNorm", activation="swiglu", bias=False,
                              params_dtype=dtype, device=dev)
    w = mlp.fc1_weight
    print(f"fc1_weight: {type(w).__name__}, logical shape {tuple(w.shape)}, dtype seen by autograd {w.dtype}")
    opt = te.FusedAdam(mlp.parameters(), lr=1e-3, master_weights=True)
    x = torch.randn(512, a.hidden, device=dev, dtype=dtype)
    target = torch.randn(512, a.hidden, device=dev, dtype=dtype)
    losses = []
    for _ in range(a.steps):
        opt.zero_grad(set_to_none=True)
        with te.autocast(enabled=True, recipe=recipe):
            y = mlp(x)
        loss = (y.float() - target.float()).square().mean()
        loss.backward()
        opt.step()
        losses.append(float(loss.detach()))
    buf = io.BytesIO()
    torch.save(mlp.state_dict(), buf)
    buf.seek(0)
    before = mlp.fc1_weight.dequantize().clone()
    mlp.load_state_dict(torch.load(buf, weights_only=False))
    same = torch.equal(before, mlp.fc1_weight.dequantize())
    print(f"{a.recipe}: loss {losses[0]:.4f} -> {losses[-1]:.4f}; state dict round trip bit-exact: {same}")
    return losses, same


if __name__ == "__main__":
    main()
