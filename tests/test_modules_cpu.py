"""Modules on the CPU reference path against plain torch.nn implementations."""
import copy
import io
import pickle

import pytest
import torch
import torch.nn.functional as TF

import transformerengine_b200 as te
from transformerengine_b200.common import recipe as R

RECIPES = {
    "delayed": lambda: R.DelayedScaling(amax_history_len=16),
    "current": lambda: R.Float8CurrentScaling(),
    "mxfp8": lambda: R.MXFP8BlockScaling(),
    "nvfp4": lambda: R.NVFP4BlockScaling(),
    "block": lambda: R.Float8BlockScaling(),
}
TOL = {"delayed": 0.08, "current": 0.08, "mxfp8": 0.08, "nvfp4": 0.3, "block": 0.08}


def rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def test_linear_matches_torch():
    m = te.Linear(64, 96, device="cpu", params_dtype=torch.float32)
    x = torch.randn(4, 8, 64, requires_grad=True)
    y = m(x)
    ref = TF.linear(x, m.weight, m.bias)
    assert rel(y, ref) < 1e-6
    y.sum().backward()
    assert rel(m.weight.grad, torch.ones(32, 96).t() @ x.detach().reshape(32, 64)) < 1e-5


@pytest.mark.parametrize("name", list(RECIPES))
def test_linear_quantized(name):
    m = te.Linear(128, 256, device="cpu", params_dtype=torch.float32)
    x = torch.randn(64, 128, requires_grad=True)
    with te.autocast(enabled=True, recipe=RECIPES[name]()):
        y = m(x)
    ref = TF.linear(x, m.weight, m.bias)
    assert rel(y, ref) < TOL[name]
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().clone().requires_grad_(True)
    w = m.weight.detach().clone().requires_grad_(True)
    TF.linear(xr, w, m.bias.detach()).backward(g)
    assert rel(x.grad, xr.grad) < TOL[name] * 1.5
    assert rel(m.weight.grad, w.grad) < TOL[name] * 1.5
    assert rel(m.bias.grad, g.sum(0)) < 1e-5


@pytest.mark.parametrize("norm", ["LayerNorm", "RMSNorm"])
@pytest.mark.parametrize("zc", [False, True])
def test_layernorm_linear(norm, zc):
    m = te.LayerNormLinear(64, 128, normalization=norm, zero_centered_gamma=zc, device="cpu",
                           params_dtype=torch.float32)
    with torch.no_grad():
        m.layer_norm_weight.add_(torch.randn(64) * 0.1)
    x = torch.randn(16, 64, requires_grad=True)
    y = m(x)
    g = m.layer_norm_weight + (1 if zc else 0)
    if norm == "LayerNorm":
        ln = TF.layer_norm(x, (64,), g, m.layer_norm_bias, 1e-5)
    else:
        ln = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-5) * g
    ref = TF.linear(ln, m.weight, m.bias)
    assert rel(y, ref) < 1e-5
    gy = torch.randn_like(y)
    gx_ref, gw_ref = torch.autograd.grad(ref, [x, m.layer_norm_weight], gy, retain_graph=True)
    y.backward(gy)
    assert rel(x.grad, gx_ref) < 1e-4 and rel(m.layer_norm_weight.grad, gw_ref) < 1e-4


@pytest.mark.parametrize("act", ["gelu", "swiglu", "relu", "geglu", "silu", "qgelu", "srelu", "reglu"])
def test_layernorm_mlp(act):
    m = te.LayerNormMLP(64, 128, activation=act, normalization="RMSNorm", device="cpu", params_dtype=torch.float32)
    x = torch.randn(32, 64, requires_grad=True)
    y = m(x)
    ln = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-5) * m.layer_norm_weight
    h = TF.linear(ln, m.fc1_weight, m.fc1_bias)
    base = {"gelu": lambda t: TF.gelu(t, approximate="tanh"), "relu": torch.relu, "silu": TF.silu,
            "qgelu": lambda t: t * torch.sigmoid(1.702 * t), "srelu": lambda t: torch.relu(t) ** 2}
    gated = {"swiglu": "silu", "geglu": "gelu", "reglu": "relu"}
    if act in gated:
        a, b = h.chunk(2, dim=-1)
        h = base[gated[act]](a) * b
    else:
        h = base[act](h)
    ref = TF.linear(h, m.fc2_weight, m.fc2_bias)
    assert rel(y, ref) < 1e-5
    gy = torch.randn_like(y)
    refs = torch.autograd.grad(ref, [x, m.fc1_weight, m.fc2_weight, m.fc1_bias], gy, retain_graph=True)
    y.backward(gy)
    for got, want in zip([x.grad, m.fc1_weight.grad, m.fc2_weight.grad, m.fc1_bias.grad], refs):
        assert rel(got, want) < 1e-4


def _torch_layer_reference(layer, x):
    """Pre-LN GPT block with the same parameters, written with torch only ([s, b, h] input)."""
    sa, mlp = layer.self_attention, layer.layernorm_mlp
    lq = sa.layernorm_qkv
    s, b, h = x.shape
    nh = sa.num_attention_heads
    d = h // nh
    ln1 = TF.layer_norm(x, (h,), lq.layer_norm_weight, lq.layer_norm_bias, 1e-5)
    w = torch.cat([lq.query_weight, lq.key_weight, lq.value_weight], 0)
    bb = torch.cat([lq.query_bias, lq.key_bias, lq.value_bias], 0)
    qkv = TF.linear(ln1, w, bb)
    q, k, v = (t.reshape(s, b, nh, d).permute(1, 2, 0, 3) for t in qkv.chunk(3, dim=-1))
    o = TF.scaled_dot_product_attention(q, k, v, is_causal=True)
    o = o.permute(2, 0, 1, 3).reshape(s, b, h)
    x1 = x + TF.linear(o, sa.proj.weight, sa.proj.bias)
    ln2 = TF.layer_norm(x1, (h,), mlp.layer_norm_weight, mlp.layer_norm_bias, 1e-5)
    f = TF.gelu(TF.linear(ln2, mlp.fc1_weight, mlp.fc1_bias), approximate="tanh")
    return x1 + TF.linear(f, mlp.fc2_weight, mlp.fc2_bias)


def make_cfg1_layer(**kw):
    """One layer of the CPU plumbing configuration: hidden 256, 4 heads, FFN 1024 GeLU, LayerNorm."""
    torch.manual_seed(0)
    init = lambda t: torch.nn.init.normal_(t, 0.0, 0.02)  # noqa: E731
    return te.TransformerLayer(256, 1024, 4, layernorm_epsilon=1e-5, hidden_dropout=0.0, attention_dropout=0.0,
                               init_method=init, output_layer_init_method=init, self_attn_mask_type="causal",
                               params_dtype=torch.float32, device="cpu", activation="gelu", **kw)


def test_transformer_layer_matches_torch_reference():
    layer = make_cfg1_layer()
    x = torch.randn(64, 2, 256, requires_grad=True)
    y = layer(x)
    ref = _torch_layer_reference(layer, x)
    assert rel(y, ref) < 1e-5
    gy = torch.randn_like(y)
    gref = torch.autograd.grad(ref, [x, layer.layernorm_mlp.fc1_weight, layer.self_attention.proj.weight], gy,
                               retain_graph=True)
    y.backward(gy)
    assert rel(x.grad, gref[0]) < 1e-4
    assert rel(layer.layernorm_mlp.fc1_weight.grad, gref[1]) < 1e-4
    assert rel(layer.self_attention.proj.weight.grad, gref[2]) < 1e-4


def test_transformer_layer_fp8_delayed_scaling_emulation():
    layer = make_cfg1_layer()
    x = torch.randn(64, 2, 256, requires_grad=True)
    ref = _torch_layer_reference(layer, x)
    rec = R.DelayedScaling(amax_history_len=16, margin=0, fp8_format=R.Format.HYBRID)
    for _ in range(3):  # the first step runs with scale 1; later steps use the recorded amax
        layer.zero_grad()
        with te.fp8_autocast(enabled=True, fp8_recipe=rec):
            y = layer(x)
        y.sum().backward()
    assert rel(y, ref) < 0.05
    st = layer.layernorm_mlp._states["scaling_fwd"]
    assert st.amax_history.shape == (16, 6) and (st.scale != 1).any()


def test_delayed_scaling_history_roll_and_scale():
    m = te.Linear(32, 32, device="cpu", params_dtype=torch.float32)
    rec = R.DelayedScaling(amax_history_len=4, amax_compute_algo="max")
    x = torch.ones(32, 32) * 2.0
    with te.autocast(enabled=True, recipe=rec):
        m(x)
    st = m._states["scaling_fwd"]
    # after exit: amax of the step moved to slot 3 (roll by -1), slot 0 cleared, scale = 448/2
    assert st.amax_history[0, 0] == 0 and st.amax_history[3, 0] == 2.0
    assert abs(st.scale[0].item() - 224.0) < 1e-3
    with te.autocast(enabled=True, recipe=rec):
        m(x * 0.5)
    assert st.amax_history[3, 0] == 1.0 and st.amax_history[2, 0] == 2.0
    assert abs(st.scale[0].item() - 224.0) < 1e-3  # max over history still 2


def test_extra_state_roundtrip_and_recipe_module_path():
    m = te.Linear(32, 64, device="cpu", params_dtype=torch.float32)
    rec = R.DelayedScaling(amax_history_len=8)
    with te.autocast(enabled=True, recipe=rec):
        m(torch.randn(32, 32)).sum().backward()
    sd = m.state_dict()
    assert "_extra_state" in sd and sd["_extra_state"].dtype == torch.uint8 and sd["_extra_state"].numel() > 0
    raw = bytes(sd["_extra_state"].numpy().tobytes())
    assert b"transformer_engine.common.recipe" in raw  # loadable by the reference library
    obj = pickle.loads(raw)
    assert set(obj) >= {"recipe", "scale_fwd", "amax_history_fwd", "scale_bwd", "amax_history_bwd",
                        "extra_fp8_variables"}
    m2 = te.Linear(32, 64, device="cpu", params_dtype=torch.float32)
    buf = io.BytesIO()
    torch.save(sd, buf)
    buf.seek(0)
    m2.load_state_dict(torch.load(buf, weights_only=False))
    with te.autocast(enabled=True, recipe=rec):
        m2(torch.randn(32, 32))
    # loaded scales were applied when the state was built (then updated once at exit)
    assert torch.equal(m2.weight, m.weight)
    # modules that never ran quantized store an empty state
    m3 = te.Linear(8, 8, device="cpu")
    assert m3.state_dict()["_extra_state"].numel() == 0
    # stateless recipes store an empty state too
    with te.autocast(enabled=True, recipe=R.MXFP8BlockScaling()):
        te.Linear(32, 32, device="cpu", params_dtype=torch.float32)(torch.randn(32, 32))


def test_unsafe_pickle_is_refused():
    m = te.Linear(8, 8, device="cpu")

    class Evil:
        def __reduce__(self):
            return (print, ("pwned",))

    blob = torch.frombuffer(bytearray(pickle.dumps({"recipe": Evil()})), dtype=torch.uint8)
    with pytest.raises(Exception):
        m.set_extra_state(blob)


def test_nested_pickle_in_tensor_storage_is_refused(tmp_path):
    """A tensor pickled by value goes through ``torch.storage._load_from_bytes``; a payload smuggled
    in that nested archive must not run, and neither may a function of the recipe module."""
    import os

    m = te.Linear(8, 8, device="cpu")
    marker = tmp_path / "pwned"

    class Evil:
        def __reduce__(self):
            return (os.system, (f"touch {marker}",))

    inner = io.BytesIO()
    torch.save(Evil(), inner)

    class Wrapper:
        def __reduce__(self):
            return (torch.storage._load_from_bytes, (inner.getvalue(),))

    blob = torch.frombuffer(bytearray(pickle.dumps({"recipe": Wrapper()})), dtype=torch.uint8)
    with pytest.raises(Exception):
        m.set_extra_state(blob)
    assert not marker.exists()
    # an attribute of the recipe module that is not a recipe class is refused as well
    payload = b"\x80\x04" + pickle.GLOBAL + b"transformer_engine.common.recipe\n_install_pickle_alias\n" + pickle.STOP
    with pytest.raises(pickle.UnpicklingError):
        m.set_extra_state(torch.frombuffer(bytearray(payload), dtype=torch.uint8))
    # honest tensors still load through the weights-only stand-in
    good = te.Linear(32, 64, device="cpu", params_dtype=torch.float32)
    with te.autocast(enabled=True, recipe=R.DelayedScaling(amax_history_len=4)):
        good(torch.randn(32, 32)).sum().backward()
    fresh = te.Linear(32, 64, device="cpu", params_dtype=torch.float32)
    fresh.set_extra_state(good.get_extra_state())
    assert isinstance(fresh.fp8_meta["recipe"], R.DelayedScaling)


def test_parameters_split_names_and_weight_cache():
    m = te.Linear(32, 96, parameters_split=("query", "key", "value"), device="cpu", params_dtype=torch.float32)
    names = dict(m.named_parameters()).keys()
    assert {"query_weight", "key_weight", "value_weight", "query_bias"} <= set(names)
    x = torch.randn(32, 32)
    with te.autocast(enabled=True, recipe=R.MXFP8BlockScaling()):
        m(x)
        first = m._weight_cache["weight"][1]
        m(x)
        assert m._weight_cache["weight"][1] is first  # unchanged weights are not re-quantized
    y = m(x)
    y.sum().backward()
    assert m.key_weight.grad is not None and m.key_weight.grad.shape == (32, 32)


def test_quantized_model_init_and_fused_adam():
    with te.quantized_model_init(enabled=True, recipe=R.MXFP8BlockScaling(), preserve_high_precision_init_val=True):
        m = te.Linear(64, 64, device="cpu", params_dtype=torch.float32)
    assert isinstance(m.weight, te.tensor.MXFP8Tensor)
    opt = te.FusedAdam(m.parameters(), lr=1e-2, master_weights=True)
    x = torch.randn(32, 64)
    with te.autocast(enabled=True, recipe=R.MXFP8BlockScaling()):
        y = m(x)
    y.pow(2).mean().backward()
    before = m.weight.dequantize().clone()
    opt.step()
    assert not torch.equal(before, m.weight.dequantize())


def test_activation_recompute_matches():
    layer = make_cfg1_layer()
    x = torch.randn(16, 2, 256, requires_grad=True)
    y = layer(x)
    y.sum().backward()
    g0, w0 = x.grad.clone(), layer.layernorm_mlp.fc2_weight.grad.clone()
    layer.zero_grad()
    x.grad = None
    for reentrant in (True, False):
        y2 = te.checkpoint(layer, x, use_reentrant=reentrant)
        y2.sum().backward()
        assert rel(x.grad, g0) < 1e-6 and rel(layer.layernorm_mlp.fc2_weight.grad, w0) < 1e-6
        layer.zero_grad()
        x.grad = None


def test_fused_adam_matches_torch_adamw():
    ps = [torch.randn(33, 7), torch.randn(128)]
    a = [p.clone().requires_grad_(True) for p in ps]
    b = [p.clone().requires_grad_(True) for p in ps]
    o1 = te.FusedAdam(a, lr=1e-2, betas=(0.9, 0.95), weight_decay=0.1)
    o2 = torch.optim.AdamW(b, lr=1e-2, betas=(0.9, 0.95), weight_decay=0.1)
    for _ in range(4):
        for p, q in zip(a, b):
            g = torch.randn_like(p)
            p.grad, q.grad = g.clone(), g.clone()
        o1.step()
        o2.step()
    for p, q in zip(a, b):
        assert rel(p, q) < 1e-5
    sd = o1.state_dict()
    o3 = te.FusedAdam(a, lr=1e-2)
    o3.load_state_dict(sd)


def test_fsdp2_hooks_reassemble_row_shards():
    """Gathering the row shards' raw bytes (and MXFP8 scale tiles) gives the quantized full tensor."""
    from transformerengine_b200.tensor.float8 import Float8CurrentScalingQuantizer
    from transformerengine_b200.tensor.mxfp8 import MXFP8Quantizer

    torch.manual_seed(0)
    w = torch.randn(256, 64)
    q = MXFP8Quantizer(columnwise=False)
    full = q(w)
    shards = [q(w[:128]), q(w[128:])]
    outs, meta = zip(*[s.fsdp_pre_all_gather() for s in shards])
    gathered = tuple(torch.cat([o[i] for o in outs]) for i in range(2))
    rebuilt, _ = shards[0].fsdp_post_all_gather(gathered, meta[0])
    assert torch.equal(rebuilt.dequantize(), full.dequantize())
    q8 = Float8CurrentScalingQuantizer(torch.float8_e4m3fn, device="cpu")
    f = q8(w)
    (data,), m8 = f.fsdp_pre_all_gather()
    rebuilt8, _ = f.fsdp_post_all_gather((torch.cat([data[:128], data[128:]]),), m8)
    assert torch.equal(rebuilt8.dequantize(), f.dequantize())


@pytest.mark.parametrize("use_reentrant", [True, False])
def test_checkpoint_is_consistent_under_delayed_scaling(use_reentrant):
    """Activation recompute quantizes with the scales of the first run and records no second amax:
    outputs, gradients and the amax histories equal the run without recompute bit for bit."""
    def run(ckpt):
        torch.manual_seed(0)
        m1 = te.Linear(32, 32, device="cpu", params_dtype=torch.float32)
        m2 = te.Linear(32, 32, device="cpu", params_dtype=torch.float32)
        rec = R.DelayedScaling(amax_history_len=4)
        seen = []
        for step in range(3):
            x = (torch.randn(16, 32) * (step + 1)).requires_grad_()
            with te.autocast(enabled=True, recipe=rec):
                if ckpt:
                    y = te.checkpoint(m2, te.checkpoint(m1, x, use_reentrant=use_reentrant),
                                      use_reentrant=use_reentrant)
                else:
                    y = m2(m1(x))
            y.square().sum().backward()
            seen.append([y.detach().clone(), m1.weight.grad.clone(), m2.weight.grad.clone(), x.grad.clone()]
                        + [m._states[k].amax_history.clone() for m in (m1, m2) for k in ("scaling_fwd", "scaling_bwd")]
                        + [m._states[k].scale.clone() for m in (m1, m2) for k in ("scaling_fwd", "scaling_bwd")])
            m1.weight.grad = m2.weight.grad = None
        return seen

    for plain, ckpt in zip(run(False), run(True)):
        for a, b in zip(plain, ckpt):
            assert torch.equal(a, b)


def test_unimplemented_options_are_refused_not_ignored():
    import transformerengine_b200 as te

    with pytest.raises(NotImplementedError):
        te.GroupedLinear(2, 16, 16, save_original_input=True, device="cpu")
    with pytest.raises(NotImplementedError):
        te.LayerNormMLP(16, 32, activation_params={"limit": 7.0}, device="cpu")
    lin = te.Linear(16, 16, device="cpu", params_dtype=torch.float32)
    with pytest.raises(NotImplementedError):
        lin(torch.randn(4, 16), fp8_output=True)
    opt = te.FusedAdam(lin.parameters(), lr=1e-3)
    with pytest.raises(NotImplementedError):
        opt.step(grad_scaler=object())


def test_transformer_layer_passes_rotary_interleaving_to_attention():
    import transformerengine_b200 as te

    torch.manual_seed(0)
    kw = dict(hidden_size=64, ffn_hidden_size=128, num_attention_heads=4, hidden_dropout=0.0, attention_dropout=0.0,
              params_dtype=torch.float32, device="cpu", fuse_qkv_params=True)
    a = te.TransformerLayer(**kw, rotary_pos_interleaved=False)
    b = te.TransformerLayer(**kw, rotary_pos_interleaved=True)
    b.load_state_dict(a.state_dict())
    assert b.self_attention.rotary_pos_interleaved and not a.self_attention.rotary_pos_interleaved
    x = torch.randn(8, 2, 64)
    freqs = te.RotaryPositionEmbedding(16)(8)
    ya, yb = a(x, rotary_pos_emb=freqs), b(x, rotary_pos_emb=freqs)
    assert not torch.allclose(ya, yb)          # the two pairings of channels rotate differently
    # the interleaved layer equals rotating with pairs (2i, 2i + 1): check through the functional form
    from transformerengine_b200.attention.rope import apply_rotary_pos_emb

    q = torch.randn(8, 2, 4, 16)
    r1 = apply_rotary_pos_emb(q, freqs, "sbhd", interleaved=True)
    r2 = apply_rotary_pos_emb(q, freqs, "sbhd", interleaved=True, fused=False)
    torch.testing.assert_close(r1, r2)


@pytest.mark.parametrize("name", ["delayed", "current", "mxfp8", "block"])
@pytest.mark.parametrize("kind", ["layernorm_linear", "layernorm_mlp", "grouped_linear", "transformer_layer"])
def test_quantized_model_init_covers_every_module(name, kind):
    """Parameters created under ``quantized_model_init`` are quantized tensors in every GEMM module, and a module
    built that way computes exactly what a high-precision module holding the dequantized values computes."""
    from transformerengine_b200.tensor.base import QuantizedTensorStorage
    rec = {"delayed": R.DelayedScaling, "current": R.Float8CurrentScaling, "mxfp8": R.MXFP8BlockScaling,
           "block": R.Float8BlockScaling}[name]()

    def build():
        torch.manual_seed(0)
        kw = dict(params_dtype=torch.float32, device="cpu")
        if kind == "layernorm_linear":
            return te.LayerNormLinear(128, 256, normalization="RMSNorm", bias=True, **kw), 1
        if kind == "layernorm_mlp":
            return te.LayerNormMLP(128, 256, normalization="RMSNorm", activation="swiglu", bias=False, **kw), 2
        if kind == "grouped_linear":
            return te.GroupedLinear(2, 128, 128, bias=False, **kw), 2
        return te.TransformerLayer(128, 256, 4, hidden_dropout=0.0, attention_dropout=0.0, fuse_qkv_params=False,
                                   **kw), 6          # query / key / value, proj, fc1, fc2

    with te.quantized_model_init(enabled=True, recipe=rec, preserve_high_precision_init_val=True):
        q, expect = build()
    ref, _ = build()
    quantized = [p for p in q.parameters() if isinstance(p, QuantizedTensorStorage)]
    assert len(quantized) == expect
    assert all(getattr(p, "_high_precision_init_val", None) is not None for p in quantized)
    with torch.no_grad():
        for p, pr in zip(q.parameters(), ref.parameters()):
            pr.copy_(p.dequantize() if isinstance(p, QuantizedTensorStorage) else p)
    x = torch.randn(32, 2, 128) if kind == "transformer_layer" else torch.randn(64, 128)
    xa, xb = x.clone().requires_grad_(), x.clone().requires_grad_()
    extra = ([32, 32],) if kind == "grouped_linear" else ()
    with te.autocast(enabled=True, recipe=rec):
        ya, yb = q(xa, *extra), ref(xb, *extra)
    ya.square().sum().backward()
    yb.square().sum().backward()
    assert torch.allclose(ya, yb, atol=1e-6)
    assert torch.allclose(xa.grad, xb.grad, atol=1e-5)
    for p, pr in zip(q.parameters(), ref.parameters()):
        assert p.grad is not None and p.grad.shape == pr.grad.shape
        assert torch.allclose(p.grad, pr.grad, atol=1e-4), float((p.grad - pr.grad).abs().max())
    # the optimizer keeps fp32 masters that start from the unrounded initial values and writes back quantized
    opt = te.FusedAdam(q.parameters(), lr=1e-2, master_weights=True)
    before = quantized[0].dequantize().clone()
    opt.step()
    assert isinstance(quantized[0], QuantizedTensorStorage) and not torch.equal(before, quantized[0].dequantize())


def test_grouped_linear_output_buffers():
    """``out`` / ``dgrad_out`` receive the forward output and the input gradient; rows past ``sum(m_splits)`` stay
    untouched."""
    torch.manual_seed(0)
    gl = te.GroupedLinear(2, 16, 24, bias=True, params_dtype=torch.float32, device="cpu", use_grouped_tensor=True)
    x = torch.randn(10, 16, requires_grad=True)
    x2 = x.detach().clone().requires_grad_()
    out, dgrad = torch.full((12, 24), 7.0), torch.full((12, 16), 7.0)
    y = gl(x, [4, 6], out=out, dgrad_out=dgrad)
    y2 = gl(x2, [4, 6])
    assert y.data_ptr() == out.data_ptr() and torch.equal(y[:10], y2) and (out[10:] == 7).all()
    y[:10].square().sum().backward()
    y2.square().sum().backward()
    assert torch.equal(x.grad, x2.grad) and torch.equal(dgrad[:10], x2.grad) and (dgrad[10:] == 7).all()
    assert x.grad.data_ptr() == dgrad.data_ptr()
    with pytest.raises(ValueError):
        gl(x, [4, 6], out=torch.empty(12, 23))
    with pytest.raises(TypeError):
        te.GroupedLinear(2, 16, 24, device="cpu", use_grouped_tensor="yes")


@pytest.mark.parametrize("dtypes", [(torch.float16, torch.float16), (torch.uint8, torch.float16),
                                    (torch.uint8, torch.uint8), (torch.bfloat16, torch.float32)])
def test_fused_adam_scaled_states(dtypes):
    """Moments stored in fp16 / FP8 bytes (with a per-tensor scale) or mixed dtypes track the fp32-state optimizer;
    the state API returns and accepts unscaled fp32 values; checkpoints hold fp32 moments."""
    def run(**kw):
        torch.manual_seed(0)
        p = torch.nn.Parameter(torch.randn(64, 32))
        opt = te.FusedAdam([p], lr=1e-2, **kw)
        for i in range(20):
            torch.manual_seed(i)
            p.grad = torch.randn(64, 32) * 0.1
            opt.step()
        return p, opt

    ref, ref_opt = run()
    p, opt = run(exp_avg_dtype=dtypes[0], exp_avg_sq_dtype=dtypes[1])
    st = opt.state[p]
    assert st["exp_avg"].dtype == dtypes[0] and st["exp_avg_sq"].dtype == dtypes[1]
    tol = 2e-2 if torch.uint8 in dtypes else 2e-3
    assert (p - ref).abs().max() < tol
    m = opt.get_unscaled_state(p, "exp_avg")
    assert m.dtype == torch.float32
    rel = (m - ref_opt.state[ref]["exp_avg"]).abs().max() / ref_opt.state[ref]["exp_avg"].abs().max()
    assert rel < (0.2 if dtypes[0] == torch.uint8 else 1e-2)     # E4M3 rounds by up to 6 % per step
    sd = opt.state_dict()
    assert sd["state"][0]["exp_avg"].dtype == torch.float32 and sd["state"][0]["exp_avg_sq"].dtype == torch.float32
    opt2 = te.FusedAdam([p], lr=1e-2, exp_avg_dtype=dtypes[0], exp_avg_sq_dtype=dtypes[1])
    opt2.load_state_dict(sd)
    torch.testing.assert_close(opt2.get_unscaled_state(p, "exp_avg_sq"), opt.get_unscaled_state(p, "exp_avg_sq"))
    # set_scaled_state: an fp32 value goes in, the stored form is scaled and rounded
    new = torch.randn(64, 32) * 3.0
    opt.set_scaled_state(p, "exp_avg", new)
    back = opt.get_unscaled_state(p, "exp_avg")
    assert (back - new).abs().max() <= (0.07 if dtypes[0] == torch.uint8 else 0.02) * new.abs().max()
    # initialize_state before any step, with master weights taken from the parameter
    q = torch.nn.Parameter(torch.randn(8, 8).bfloat16())
    o3 = te.FusedAdam([q], master_weights=True, exp_avg_dtype=dtypes[0], exp_avg_sq_dtype=dtypes[1])
    o3.initialize_state(q)
    assert torch.equal(o3.get_unscaled_state(q, "master_param"), q.detach().float())
    assert float(o3.get_unscaled_state(q, "exp_avg").abs().max()) == 0.0


def _mx(t):
    from transformerengine_b200.tensor.mxfp8 import MXFP8Quantizer
    return MXFP8Quantizer()(t.detach()).dequantize()


@pytest.mark.parametrize("override", ["high_precision", "dequantized"])
def test_backward_override_runs_the_backward_gemms_unquantized(override):
    """``recipe.backward_override``: the forward pass is the quantized one, the backward GEMMs take the original
    operands (``high_precision``) or the dequantized forward operands (``dequantized``), unquantized."""
    torch.manual_seed(0)
    pick = (lambda t: t.detach()) if override == "high_precision" else _mx
    rec, plain = R.MXFP8BlockScaling(backward_override=override), R.MXFP8BlockScaling()
    x = torch.randn(32, 64)

    def run(m, recipe):
        xi = x.clone().requires_grad_()
        m.zero_grad()
        with te.autocast(enabled=True, recipe=recipe):
            y = m(xi)
        y.square().sum().backward()
        return y.detach(), xi.grad

    lin = te.Linear(64, 96, bias=True, params_dtype=torch.float32, device="cpu")
    y0, _ = run(lin, plain)
    y, gx = run(lin, rec)
    dy = 2 * y
    assert torch.equal(y, y0)
    torch.testing.assert_close(gx, dy @ pick(lin.weight))
    torch.testing.assert_close(lin.weight.grad, dy.t() @ pick(x))
    torch.testing.assert_close(lin.bias.grad, dy.sum(0))

    lnl = te.LayerNormLinear(64, 96, normalization="RMSNorm", bias=False, params_dtype=torch.float32, device="cpu")
    y0, _ = run(lnl, plain)
    y, gx = run(lnl, rec)
    assert torch.equal(y, y0)
    ln = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + lnl.eps) * lnl.layer_norm_weight.detach()
    torch.testing.assert_close(lnl.weight.grad, (2 * y).t() @ pick(ln), rtol=1e-4, atol=1e-5)

    # LayerNormMLP against autograd through a straight-through emulation: forward values of the quantized run,
    # gradients of the unquantized products
    mlp = te.LayerNormMLP(64, 128, normalization="RMSNorm", activation="gelu", bias=True, params_dtype=torch.float32,
                          device="cpu")
    y0, _ = run(mlp, plain)
    y, gx = run(mlp, rec)
    assert torch.equal(y, y0)
    w1, b1, w2, b2, g = (p.detach().clone().requires_grad_() for p in (mlp.fc1_weight, mlp.fc1_bias, mlp.fc2_weight,
                                                                        mlp.fc2_bias, mlp.layer_norm_weight))
    xi = x.clone().requires_grad_()
    ln = xi * torch.rsqrt(xi.pow(2).mean(-1, keepdim=True) + mlp.eps) * g
    sel = (lambda t: t) if override == "high_precision" else (lambda t: t + (_mx(t) - t).detach())

    def ste_linear(a, w, b):
        hp = sel(a) @ sel(w).t() + b
        return hp + ((_mx(a) @ _mx(w).t() + b) - hp).detach()

    fc1 = ste_linear(ln, w1, b1)
    act = fc1 * (0.5 + 0.5 * torch.tanh(fc1 * (0.79788456 + 0.03567741 * fc1 * fc1)))
    out = ste_linear(act, w2, b2)
    torch.testing.assert_close(out.detach(), y, rtol=1e-4, atol=1e-5)
    out.square().sum().backward()
    torch.testing.assert_close(gx, xi.grad, rtol=1e-3, atol=1e-4)
    torch.testing.assert_close(mlp.fc1_weight.grad, w1.grad, rtol=1e-3, atol=1e-4)
    torch.testing.assert_close(mlp.fc2_weight.grad, w2.grad, rtol=1e-3, atol=1e-4)
    torch.testing.assert_close(mlp.fc1_bias.grad, b1.grad, rtol=1e-3, atol=1e-4)

    # GroupedLinear: slabs of 32 rows (quantized one by one) and of 128 rows (quantized as one tensor)
    for rows in (32, 128):
        gl = te.GroupedLinear(2, 64, 96, bias=True, params_dtype=torch.float32, device="cpu")
        xg = torch.randn(2 * rows, 64)

        def run_g(recipe):
            xi = xg.clone().requires_grad_()
            gl.zero_grad()
            with te.autocast(enabled=True, recipe=recipe):
                y = gl(xi, [rows, rows])
            y.square().sum().backward()
            return y.detach(), xi.grad

        y0, _ = run_g(plain)
        y, gx = run_g(rec)
        assert torch.equal(y, y0)
        dy = 2 * y
        for g, w in enumerate((gl.weight0, gl.weight1)):
            sl = slice(g * rows, (g + 1) * rows)
            torch.testing.assert_close(gx[sl], dy[sl] @ pick(w), rtol=1e-4, atol=1e-5)
            torch.testing.assert_close(w.grad, dy[sl].t() @ pick(xg[sl]), rtol=1e-4, atol=1e-5)
        torch.testing.assert_close(gl.bias1.grad, dy[rows:].sum(0), rtol=1e-4, atol=1e-5)


def test_layernorm_mlp_clamped_swiglu_and_glu():
    """``activation="clamped_swiglu"`` with ``activation_params`` (the GPT-OSS gated unit) and ``"glu"``: forward
    and gradients against autograd through the formulas."""
    torch.manual_seed(0)
    x = torch.randn(16, 32) * 3
    for act, params in (("clamped_swiglu", dict(limit=2.0, alpha=1.5, glu_linear_offset=0.5)), ("clamped_swiglu", None),
                        ("glu", None)):
        mlp = te.LayerNormMLP(32, 64, normalization="RMSNorm", activation=act, activation_params=params, bias=False,
                              params_dtype=torch.float32, device="cpu")
        assert mlp.fc1_weight.shape == (128, 32)
        xi = x.clone().requires_grad_()
        y = mlp(xi)
        y.square().sum().backward()
        xr = x.clone().requires_grad_()
        g, w1, w2 = (p.detach().clone().requires_grad_() for p in (mlp.layer_norm_weight, mlp.fc1_weight, mlp.fc2_weight))
        ln = xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + mlp.eps) * g
        a, b = (ln @ w1.t()).chunk(2, dim=-1)
        if act == "glu":
            h = torch.sigmoid(a) * b
        else:
            p = dict(limit=7.0, alpha=1.702, glu_linear_offset=1.0)
            p.update(params or {})
            ac = a.clamp(max=p["limit"])
            h = ac * torch.sigmoid(p["alpha"] * ac) * (b.clamp(-p["limit"], p["limit"]) + p["glu_linear_offset"])
        want = h @ w2.t()
        want.square().sum().backward()
        torch.testing.assert_close(y, want, rtol=1e-4, atol=1e-5)
        torch.testing.assert_close(xi.grad, xr.grad, rtol=1e-3, atol=1e-4)
        torch.testing.assert_close(mlp.fc1_weight.grad, w1.grad, rtol=1e-3, atol=1e-4)
    with pytest.raises(NotImplementedError):
        te.LayerNormMLP(32, 64, activation="swiglu", activation_params=dict(limit=1.0), device="cpu")
    with pytest.raises(ValueError):
        te.LayerNormMLP(32, 64, activation="clamped_swiglu", activation_params=dict(beta=1.0), device="cpu")


@pytest.mark.parametrize("kind", ["LayerNorm", "RMSNorm", "Linear", "LayerNormLinear", "LayerNormMLP", "GroupedLinear",
                                  "MultiheadAttention", "TransformerLayer"])
def test_deferred_init_on_the_meta_device(kind):
    """``device="meta"`` builds a module without memory; ``reset_parameters()`` materialises and initialises it
    (test model: the reference's ``tests/pytorch/test_deferred_init.py``)."""
    import copy
    import pickle
    args, kw = {"LayerNorm": ((64,), {}), "RMSNorm": ((64,), {}), "Linear": ((64, 128), dict(bias=True)),
                "LayerNormLinear": ((64, 128), dict(bias=True)), "LayerNormMLP": ((64, 128), dict(bias=True)),
                "GroupedLinear": ((2, 64, 64), dict(bias=True)),
                "MultiheadAttention": ((64, 4), dict(fuse_qkv_params=True)),
                "TransformerLayer": ((64, 128, 4), dict(fuse_qkv_params=False, hidden_dropout=0.0,
                                                        attention_dropout=0.0))}[kind]
    cls = getattr(te, kind)
    init = lambda t: torch.nn.init.normal_(t, 0.0, 0.5)  # noqa: E731
    if kind not in ("LayerNorm", "RMSNorm"):
        kw = dict(kw, init_method=init)
    m = cls(*args, params_dtype=torch.float32, device="meta", **kw)
    assert all(p.device.type == "meta" for p in m.parameters())
    for sub in m.modules():
        if hasattr(sub, "reset_parameters"):
            sub.reset_parameters()
    assert all(p.device.type != "meta" for p in m.parameters()), [n for n, p in m.named_parameters() if p.is_meta]
    for name, p in m.named_parameters():
        if "layer_norm_weight" in name or name.endswith("norm.weight") or (kind in ("LayerNorm", "RMSNorm") and name == "weight"):
            assert (p == 1).all(), name
        elif "bias" in name:
            assert (p == 0).all(), name
        elif "weight" in name and p.dim() == 2 and "proj" not in name and "fc2" not in name:
            assert 0.4 < float(p.detach().std()) < 0.6, name
    x = torch.randn(8, 2, 64) if kind in ("MultiheadAttention", "TransformerLayer") else torch.randn(16, 64)
    y = m(x, [8, 8]) if kind == "GroupedLinear" else m(x)
    assert torch.isfinite(y if isinstance(y, torch.Tensor) else y[0]).all()
    # re-initialising a live module keeps the statistics; copies and pickles still work
    stats = {n: (float(p.detach().mean()), float(p.detach().std())) for n, p in m.named_parameters() if p.dim() == 2}
    for sub in m.modules():
        if hasattr(sub, "reset_parameters"):
            sub.reset_parameters()
    for n, p in m.named_parameters():
        if p.dim() == 2:
            assert abs(float(p.detach().std()) - stats[n][1]) < 0.1 * max(stats[n][1], 1e-3), n
    copy.deepcopy(m)
    pickle.loads(pickle.dumps(m))


def test_deferred_init_with_quantized_parameters():
    from transformerengine_b200.tensor.base import QuantizedTensorStorage
    rec = R.MXFP8BlockScaling()
    with te.quantized_model_init(enabled=True, recipe=rec):
        lin = te.Linear(128, 128, bias=False, params_dtype=torch.float32, device="meta")
    assert lin.weight.is_meta
    lin.reset_parameters()
    assert isinstance(lin.weight, QuantizedTensorStorage) and not lin.weight.is_meta
    assert 0.015 < float(lin.weight.dequantize().std()) < 0.03
    with te.autocast(enabled=True, recipe=rec):
        assert torch.isfinite(lin(torch.randn(32, 128))).all()
    before = lin.weight.dequantize().clone()
    lin.reset_parameters()                     # a quantized parameter is re-drawn and re-quantized in place
    assert not torch.equal(before, lin.weight.dequantize())


@pytest.mark.parametrize("kind", ["Linear", "LayerNormLinear", "LayerNormMLP", "GroupedLinear"])
def test_delayed_weight_gradients(kind):
    """``delay_wgrad_compute``: the backward pass returns the input gradient and postpones the weight-gradient
    GEMMs until ``backward_dw()`` (zero-bubble pipeline schedules)."""
    def build(delay):
        torch.manual_seed(0)
        kw = dict(params_dtype=torch.float32, device="cpu", delay_wgrad_compute=delay, bias=True)
        return {"Linear": lambda: te.Linear(32, 64, **kw), "LayerNormLinear": lambda: te.LayerNormLinear(32, 64, **kw),
                "LayerNormMLP": lambda: te.LayerNormMLP(32, 64, **kw),
                "GroupedLinear": lambda: te.GroupedLinear(2, 32, 64, **kw)}[kind]()

    a, b = build(True), build(False)
    x = torch.randn(64, 32)
    xa, xb = x.clone().requires_grad_(), x.clone().requires_grad_()
    extra = ([32, 32],) if kind == "GroupedLinear" else ()
    with te.autocast(enabled=True, recipe=R.MXFP8BlockScaling()):
        ya, yb = a(xa, *extra), b(xb, *extra)
    ya.square().sum().backward()
    yb.square().sum().backward()
    assert a.need_backward_dw() and not b.need_backward_dw()
    assert torch.equal(xa.grad, xb.grad)
    weights = [p for p in a.parameters() if p.dim() == 2]
    assert all(p.grad is None for p in weights)
    a.backward_dw()
    for (n, pa), (_, pb) in zip(a.named_parameters(), b.named_parameters()):
        torch.testing.assert_close(pa.grad, pb.grad, msg=n)
