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


@pytest.mark.parametrize("opts", [dict(retain_pinned_cpu_buffers=True), dict(double_buffering=True),
                                  dict(manual_synchronization=True),
                                  dict(retain_pinned_cpu_buffers=True, double_buffering=True)])
def test_cpu_offload_options_on_gpu(opts):
    """Pinned-buffer pool, double-buffered reloads and manual control of the copies: same gradients as without
    offloading over three iterations; the pool stops allocating after the first iteration."""
    import transformerengine_b200 as te

    torch.manual_seed(3)
    layers = [te.Linear(512, 512, bias=False, params_dtype=torch.bfloat16, device="cuda") for _ in range(4)]
    res = te.get_cpu_offload_context(enabled=True, num_layers=3, model_layers=4, **opts)
    ctx, sync = res[0], res[1]
    manual = res[2] if len(res) > 2 else None
    allocs = []
    for it in range(3):
        x = torch.randn(512, 512, device="cuda", dtype=torch.bfloat16, requires_grad=True)
        h = x
        for i, l in enumerate(layers):
            with ctx:
                h = torch.tanh(l(h))
            h = sync(h)
            if manual is not None:
                manual.start_offload_layer(i)
                manual.release_activation_forward_gpu_memory(i)
        if manual is not None:
            manual.start_reload_layer(2)
        h.float().sum().backward()
        ref = x.detach().clone().requires_grad_()
        hr = ref
        for l in layers:
            hr = torch.tanh(l(hr))
        hr.float().sum().backward()
        torch.cuda.synchronize()
        assert torch.equal(x.grad, ref.grad), (opts, it)
        assert not ctx.handler.store
        allocs.append(ctx.handler.host_allocations)
    if opts.get("retain_pinned_cpu_buffers"):
        assert allocs[1] == allocs[0] and allocs[2] == allocs[0]
    else:
        assert allocs[2] > allocs[0]


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


def test_bounded_wait_expires_and_reports():
    """A wait on a flag that nothing sets gives up after its limit, records the peer-flag status code and
    returns: the context stays usable (the benign form of a lost peer)."""
    import transformerengine_b200 as te
    from transformerengine_b200.ops import _ext

    C = _ext.get()
    dev = torch.cuda.current_device()
    st = C.status(dev)
    st.zero_()
    flags = torch.zeros(8, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    C.ep_wait(flags.data_ptr(), 4, 1, st, limit_cycles=2_000_000)   # about a millisecond of SM clocks
    t1.record()
    torch.cuda.synchronize()
    assert t0.elapsed_time(t1) < 200.0
    assert int(st[0].item()) == 4  # kTimeoutPeerFlag
    with pytest.raises(RuntimeError, match="peer flag"):
        te.check_status()
    te.check_status()  # the status word was cleared by the failed check
    # a flag that IS set lets the wait through, and kernels keep running on the same context
    flags.fill_(1)
    C.ep_wait(flags.data_ptr(), 4, 1, st, limit_cycles=2_000_000)
    torch.cuda.synchronize()
    te.check_status()
    assert torch.ones(4, device="cuda").sum().item() == 4.0


def test_graphed_callables_pipeline_order_and_weight_caching():
    """Two model chunks, two micro-batches, captured in a 1F1B-like order from one pool; weights quantized
    outside the forward graphs and refreshed in place when they change."""
    import transformerengine_b200 as te

    torch.manual_seed(0)
    recipe = te.recipe.MXFP8BlockScaling()
    chunks = [te.Linear(256, 256, bias=False, params_dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    xs = [torch.randn(128, 256, device="cuda", dtype=torch.bfloat16) for _ in range(2)]

    def eager(mbs):
        for c in chunks:
            c.zero_grad(set_to_none=True)
        outs = []
        for x in mbs:
            with te.autocast(enabled=True, recipe=recipe):
                y = chunks[1](chunks[0](x.clone().requires_grad_()))
            y.float().sum().backward()
            outs.append(y.detach().clone())
        return outs, [c.weight.grad.detach().clone() for c in chunks]

    ref_out, ref_grad = eager(xs)
    for c in chunks:
        c.zero_grad(set_to_none=True)
    sample = [(xs[mb].clone().requires_grad_(),) for mb in range(2) for _ in range(2)]
    g0, g1 = te.make_graphed_callables(tuple(chunks), sample, num_warmup_iters=2, enabled=True, recipe=recipe,
                                       cache_quantized_params=True, _order=[1, 2, 1, 2, -2, -1, -2, -1])
    for c in chunks:
        c.zero_grad(set_to_none=True)

    def graphed(mbs, first):
        outs = []
        hs = []
        for i, x in enumerate(mbs):
            h = g0(x.clone().requires_grad_(), is_first_microbatch=first and i == 0)
            hs.append(g1(h, is_first_microbatch=first and i == 0))
        for y in hs:
            y.float().sum().backward()
            outs.append(y.detach().clone())
        return outs

    out = graphed(xs, True)
    torch.cuda.synchronize()
    te.check_status()
    for a, b in zip(out, ref_out):
        assert torch.allclose(a.float(), b.float(), atol=2e-2, rtol=2e-2)
    for c, g in zip(chunks, ref_grad):
        assert torch.allclose(c.weight.grad.float(), g.float(), atol=5e-2, rtol=5e-2)
    # change the weights: without a refresh the graphs keep the cached FP8 weights, with it they follow
    with torch.no_grad():
        for c in chunks:
            c.weight.mul_(2.0)
    stale = graphed(xs, False)
    fresh = graphed(xs, True)
    torch.cuda.synchronize()
    assert torch.allclose(stale[0].float(), ref_out[0].float(), atol=2e-2, rtol=2e-2)
    assert torch.allclose(fresh[0].float(), 4.0 * ref_out[0].float(), atol=8e-2, rtol=3e-2)


def test_fused_adam_capturable_and_param_remainders():
    import transformerengine_b200 as te

    torch.manual_seed(0)
    shapes = [(257, 33), (1024,), (64, 64)]
    base = [torch.randn(s, device="cuda", dtype=torch.bfloat16) for s in shapes]
    grads = [[torch.randn(s, device="cuda", dtype=torch.bfloat16) for s in shapes] for _ in range(4)]

    def run(**kw):
        ps = [torch.nn.Parameter(b.clone()) for b in base]
        opt = te.FusedAdam(ps, lr=1e-2, betas=(0.9, 0.95), weight_decay=0.1, master_weights=True, **kw)
        for gs in grads:
            for p, g in zip(ps, gs):
                p.grad = g.clone()
            opt.step()
        torch.cuda.synchronize()
        return ps, opt

    ref, _ = run()
    cap, opt_c = run(capturable=True)
    assert isinstance(opt_c.param_groups[0]["step"], torch.Tensor) and int(opt_c.param_groups[0]["step"].item()) == 4
    rem, opt_r = run(store_param_remainders=True)
    for a, b, c in zip(ref, cap, rem):
        assert torch.equal(a, b)                      # device step counter: same update
        assert (a.float() - c.float()).abs().max().item() <= 2.0 ** -7 * a.float().abs().max().item() + 1e-6
    # the bf16 parameter and its remainder rebuild the fp32 master exactly
    st = opt_r.state[rem[0]]
    assert "param_remainder" in st and "master_param" not in st
    from transformerengine_b200.ops.misc import join_param_remainder

    master_ref = run()[1].state  # fp32 masters of a plain run
    m = join_param_remainder(rem[0].data, st["param_remainder"])
    other = list(master_ref.values())[0]["master_param"]
    assert torch.allclose(m, other, atol=1e-6, rtol=1e-6)
    # strided or expanded gradients are made dense instead of being read out of bounds
    p = torch.nn.Parameter(torch.zeros(8, 16, device="cuda", dtype=torch.bfloat16))
    o = te.FusedAdam([p], lr=1e-2, master_weights=True)
    p.grad = torch.ones(1, device="cuda", dtype=torch.bfloat16).expand(8, 16)
    o.step()
    torch.cuda.synchronize()
    assert torch.isfinite(p.float()).all() and (p != 0).all()


def test_compile_ops_trace_the_kernels_as_single_nodes_on_gpu():
    """A norm -> linear -> SwiGLU -> linear block through the ``torch.library`` operators, compiled as one graph
    (no graph breaks) in bf16 on the GPU: forward and gradients against eager PyTorch."""
    import transformerengine_b200.compile_ops as cops

    torch.manual_seed(4)
    x = torch.randn(256, 512, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    g = torch.ones(512, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w1 = (torch.randn(1024, 512, device="cuda", dtype=torch.bfloat16) * 0.05).requires_grad_()
    w2 = (torch.randn(512, 512, device="cuda", dtype=torch.bfloat16) * 0.05).requires_grad_()

    def block(x, g, w1, w2):
        return cops.linear(cops.swiglu(cops.linear(cops.rmsnorm(x, g, 1e-5), w1)), w2)

    y = torch.compile(block, backend="aot_eager", fullgraph=True)(x, g, w1, w2)
    xf = x.float()
    h = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * g.float()).to(torch.bfloat16)
    u = (h.float() @ w1.float().t()).to(torch.bfloat16).float()
    a = (torch.nn.functional.silu(u[:, :512]) * u[:, 512:]).to(torch.bfloat16)
    ref = a.float() @ w2.float().t()
    assert ((y.float() - ref).norm() / ref.norm()) < 2e-2
    y.float().sum().backward()
    assert all(t.grad is not None and torch.isfinite(t.grad).all() for t in (x, g, w1, w2))
