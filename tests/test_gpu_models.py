"""Whole-model steps on the GPU under every recipe (Llama-architecture, head dim 128 so that the
attention kernels of this library run)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("recipe_name", [None, "MXFP8BlockScaling", "NVFP4BlockScaling", "DelayedScaling",
                                         "Float8CurrentScaling", "Float8BlockScaling"])
def test_llama_tiny_trains_under_recipe(recipe_name):
    import transformerengine_b200 as te
    from transformerengine_b200.models import llama

    torch.manual_seed(0)
    cfg = llama.LlamaConfig.tiny(hidden_size=512, num_heads=4, num_kv_heads=2, ffn_hidden_size=1024)
    model = llama.LlamaModel(cfg).cuda()
    opt = te.FusedAdam(model.parameters(), lr=1e-3, master_weights=True)
    recipe = getattr(te.recipe, recipe_name)() if recipe_name else None
    tokens = torch.randint(0, cfg.vocab_size, (2, 256), device="cuda")
    losses = []
    for _ in range(4):
        opt.zero_grad(set_to_none=True)
        with te.autocast(enabled=recipe is not None, recipe=recipe):
            loss = model(tokens, labels=tokens)
        loss.backward()
        opt.step()
        losses.append(loss.item())
    te.ops.check_status()
    assert all(torch.isfinite(torch.tensor(l)) for l in losses), losses
    assert losses[-1] < losses[0], losses  # the same batch four times: the loss must fall


def test_llama_recompute_matches_plain():
    import transformerengine_b200 as te
    from transformerengine_b200.models import llama

    cfg = llama.LlamaConfig.tiny(hidden_size=512, num_heads=4, num_kv_heads=2, ffn_hidden_size=1024)
    tokens = torch.randint(0, cfg.vocab_size, (1, 256), device="cuda")
    grads = []
    for rec in (False, True):
        torch.manual_seed(0)
        cfg.recompute = rec
        model = llama.LlamaModel(cfg).cuda()
        with te.autocast(enabled=True, recipe=te.recipe.MXFP8BlockScaling()):
            loss = model(tokens, labels=tokens)
        loss.backward()
        grads.append(torch.cat([p.grad.float().reshape(-1) for p in model.parameters()]))
    te.ops.check_status()
    assert torch.allclose(grads[0], grads[1], atol=1e-3, rtol=1e-2)
