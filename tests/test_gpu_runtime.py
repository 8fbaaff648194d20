"""Runtime features on the GPU: CUDA-graph callables, activation offload, KV cache with the
library's attention kernels."""
from collections import OrderedDict

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_cpu_offload_on_gpu():
    import transformerengine_b200 as te

    torch.manual_seed(1)
    layers = [te.Linear(512, 512, bias=False, params_dtype=torch.bfloat16, device="cuda") for _ in range(3)]
    x = torch.randn(512, 512, device="cuda", dtype=torch.bfloat16, requires_grad=True)

    def run(offload):
        ctx, sync = te.get_cpu_offload_context(enabled=offload, num_layers=2, model_layers=3)
        h = x
        for l in layers:
            with ctx:
                h = torch.tanh(l(h))
            h = sync(h)
        h.float().sum().backward()
        g = x.grad.clone()
        x.grad = None
        return g, ctx

    g0, _ = run(False)
    g1, ctx = run(True)
    torch.cuda.synchronize()
    assert ctx.handler.bytes_offloaded > 0
    assert torch.equal(g0, g1)


def test_kv_cache_decoding_with_attention_kernels():
    import transformerengine_b200 as te

    torch.manual_seed(2)
    b, h, hk, d, total = 2, 4, 2, 128, 160
    mha = te.MultiheadAttention(h * d, h, num_gqa_groups=hk, attention_dropout=0.0, attn_mask_type="causal",
                                qkv_format="bshd", bias=False, params_dtype=torch.bfloat16, device="cuda")
    mha.eval()
    rope = te.RotaryPositionEmbedding(d)(total).cuda()
    x = torch.randn(b, total, h * d, device="cuda", dtype=torch.bfloat16) * 0.5
    with torch.no_grad():
        full = mha(x, rotary_pos_emb=rope)
        params = te.InferenceParams(max_batch_size=2, max_sequence_length=256, num_heads_kv=hk, head_dim_k=d,
                                    dtype=torch.bfloat16, is_paged=True, page_size=64, total_num_pages=16,
                                    qkv_format="bshd")
        outs, pos = [], 0
        for n in (128, 16, 8, 8):
            params.pre_step(OrderedDict((i, n) for i in range(b)))
            outs.append(mha(x[:, pos:pos + n], rotary_pos_emb=rope, inference_params=params))
            pos += n
        inc = torch.cat(outs, dim=1)
    te.check_status()
    err = (inc.float() - full.float()).abs().max().item()
    assert err < 5e-2 * max(full.float().abs().max().item(), 1.0), err


@pytest.mark.parametrize("quantized", [False, True])
def test_graphed_callable_matches_eager(quantized):
    import transformerengine_b200 as te

    torch.manual_seed(0)
    recipe = te.recipe.MXFP8BlockScaling() if quantized else None
    mod = te.LayerNormMLP(256, 512, bias=False, normalization="RMSNorm", activation="swiglu",
                          params_dtype=torch.bfloat16, device="cuda")
    x = torch.randn(128, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    with te.autocast(enabled=quantized, recipe=recipe):
        ref = mod(x)
    ref.float().sum().backward()
    gx_ref = x.grad.clone()
    gw_ref = mod.fc1_weight.grad.clone()
    ref = ref.detach()  # drop the eager autograd graph: its AccumulateGrad nodes are bound to the default stream
    x.grad = None
    mod.zero_grad(set_to_none=True)
    graphed = te.make_graphed_callables(mod, (x.detach().clone().requires_grad_(),), num_warmup_iters=2,
                                        enabled=quantized, recipe=recipe)
    mod.zero_grad(set_to_none=True)
    for _ in range(2):  # replay twice with the same input: results must repeat
        x2 = x.detach().clone().requires_grad_()
        out = graphed(x2)
        out.float().sum().backward()
    torch.cuda.synchronize()
    te.check_status()
    assert torch.allclose(out.float(), ref.float(), atol=2e-2, rtol=2e-2)
    assert torch.allclose(x2.grad.float(), gx_ref.float(), atol=3e-2, rtol=3e-2)
    assert torch.isfinite(mod.fc1_weight.grad.float()).all() and gw_ref.shape == mod.fc1_weight.grad.shape
