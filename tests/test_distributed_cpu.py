"""Tensor parallel + sequence parallel over gloo (2 CPU ranks) against the unsharded layer."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import transformerengine_b200 as te
from transformerengine_b200.common import recipe as R


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _make_layer(tp_group=None, tp=1):
    torch.manual_seed(0)
    init = lambda t: torch.nn.init.normal_(t, 0.0, 0.02)  # noqa: E731
    return te.TransformerLayer(256, 1024, 4, layernorm_epsilon=1e-5, hidden_dropout=0.0, attention_dropout=0.0,
                               init_method=init, output_layer_init_method=init, self_attn_mask_type="causal",
                               params_dtype=torch.float32, device="cpu", activation="gelu", tp_group=tp_group,
                               tp_size=tp, set_parallel_mode=tp > 1, sequence_parallel=tp > 1)


def _shard(full, name, rank, tp):
    """Slice of the unsharded parameter that rank `rank` owns."""
    col = ("query_weight", "key_weight", "value_weight", "query_bias", "key_bias", "value_bias", "fc1_weight",
           "fc1_bias")
    row = ("proj.weight", "fc2_weight")
    if name.endswith(col):
        return full.chunk(tp, dim=0)[rank]
    if name.endswith(row):
        return full.chunk(tp, dim=1)[rank]
    return full


def _worker(rank, tp, port, use_fp8, q):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=tp)
    try:
        full = _make_layer()
        layer = _make_layer(dist.group.WORLD, tp)
        fp = dict(full.named_parameters())
        with torch.no_grad():
            for n, p in layer.named_parameters():
                p.copy_(_shard(fp[n], n, rank, tp))
        torch.manual_seed(1)
        x = torch.randn(64, 2, 256)
        gy = torch.randn(64, 2, 256)
        rec = R.DelayedScaling(amax_history_len=16)
        override = use_fp8 if isinstance(use_fp8, str) else None
        if override is not None:
            # quantized forward, 16-bit backward GEMMs: MXFP8 blocks run along the contraction dim, which both
            # shardings leave whole, so sharded and unsharded layers see the same rounded operands
            rec, use_fp8 = R.MXFP8BlockScaling(backward_override=override), True
        xs = x.chunk(tp, dim=0)[rank].clone().requires_grad_(True)
        xf = x.clone().requires_grad_(True)
        with te.autocast(enabled=use_fp8, recipe=rec, amax_reduction_group=dist.group.WORLD):
            y = layer(xs)
        y.backward(gy.chunk(tp, dim=0)[rank])
        with te.autocast(enabled=use_fp8, recipe=rec):
            yf = full(xf)
        yf.backward(gy)
        tol = 2e-3 if override else (0.06 if use_fp8 else 1e-5)

        def rel(a, b):
            return ((a - b).norm() / (b.norm() + 1e-12)).item()

        errs = {"out": rel(y, yf.chunk(tp, dim=0)[rank]), "dx": rel(xs.grad, xf.grad.chunk(tp, dim=0)[rank])}
        lp = dict(layer.named_parameters())
        for n in ("layernorm_mlp.fc1_weight", "layernorm_mlp.fc2_weight", "self_attention.proj.weight",
                  "self_attention.layernorm_qkv.key_weight"):
            errs[n] = rel(lp[n].grad, _shard(fp[n].grad, n, rank, tp))
        # parameters replicated over TP but fed sequence shards: their gradient is summed by the trainer
        g = lp["layernorm_mlp.layer_norm_weight"].grad.clone()
        dist.all_reduce(g)
        errs["ln_w"] = rel(g, fp["layernorm_mlp.layer_norm_weight"].grad)
        assert getattr(lp["layernorm_mlp.layer_norm_weight"], "sequence_parallel", False)
        bad = {k: v for k, v in errs.items() if not v < tol}
        q.put((rank, bad))
    except Exception as e:  # noqa: BLE001
        import traceback
        q.put((rank, {"exception": traceback.format_exc()[-1500:]}))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("use_fp8", [False, True, "high_precision", "dequantized"])
def test_tp2_sequence_parallel_matches_unsharded(use_fp8):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, use_fp8, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    for rank, bad in res:
        assert not bad, f"rank {rank}: {bad}"


def _gather_worker(rank, world, port, q):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        from transformerengine_b200.parallel import distributed as D
        from transformerengine_b200.tensor import MXFP8Quantizer
        from transformerengine_b200.tensor.blockwise import Float8BlockQuantizer
        from transformerengine_b200.tensor.float8 import Float8Quantizer
        from transformerengine_b200.tensor.nvfp4 import NVFP4Quantizer

        torch.manual_seed(100 + rank)
        R, C = 128, 256
        x = torch.randn(R, C)
        full = torch.empty(world * R, C)
        dist.all_gather_into_tensor(full, x)
        bad = {}

        def check(name, qt, atol):
            g = D.gather_quantized_along_first_dim(qt, None)
            # the gathered tensor dequantizes to the gathered dequantized pieces, through either copy
            want = torch.empty(world * R, C)
            dist.all_gather_into_tensor(want, qt.dequantize(dtype=torch.float32).contiguous())
            got = g.dequantize(dtype=torch.float32)
            if got.shape != want.shape or (got - want).abs().max() > atol:
                bad[name + " rowwise"] = float((got - want).abs().max())
            g.update_usage(rowwise_usage=False)
            got_c = g.dequantize(dtype=torch.float32)
            ref_c = qt
            ref_c.update_usage(rowwise_usage=False)
            want_c = torch.empty(world * R, C)
            dist.all_gather_into_tensor(want_c, ref_c.dequantize(dtype=torch.float32).contiguous())
            if (got_c - want_c).abs().max() > atol:
                bad[name + " columnwise"] = float((got_c - want_c).abs().max())

        # per-tensor FP8: the same scale everywhere (as after an amax reduction over the group)
        amax = full.abs().max().reshape(1)
        scale = (448.0 / amax).float()
        fq = Float8Quantizer(scale, torch.zeros(1), torch.float8_e4m3fn, rowwise=True, columnwise=True)
        check("float8", fq(x), 0.0)
        check("mxfp8", MXFP8Quantizer(rowwise=True, columnwise=True)(x), 0.0)
        for dim in (1, 2):
            check(f"block{dim}d", Float8BlockQuantizer(rowwise=True, columnwise=True, block_scaling_dim=dim)(x), 0.0)
        nq = NVFP4Quantizer(rowwise=True, columnwise=True, with_amax_reduction=True, amax_reduction_group=dist.group.WORLD)
        check("nvfp4", nq(x), 0.0)
        q.put((rank, bad, None))
    except Exception:  # noqa: BLE001
        import traceback

        q.put((rank, {}, traceback.format_exc()))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def test_quantized_tensors_are_gathered_without_dequantizing():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_gather_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    for rank, bad, tb in res:
        assert tb is None, tb
        assert not bad, f"rank {rank}: {bad}"


def _ln_gathered_worker(rank, world, port, q):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        torch.manual_seed(0)
        x = torch.randn(8 * world, 32)
        bad = {}
        for kind in ("linear", "mlp"):
            torch.manual_seed(1)
            kw = dict(normalization="RMSNorm", params_dtype=torch.float32, device="cpu", tp_group=dist.group.WORLD,
                      sequence_parallel=True, return_layernorm_output=True, return_layernorm_output_gathered=True)
            if kind == "linear":
                m = te.LayerNormLinear(32, 16 * world, parallel_mode="column", bias=False, **kw)
            else:
                m = te.LayerNormMLP(32, 16 * world, set_parallel_mode=True, bias=False, **kw)
            g = m.layer_norm_weight.detach()
            xs = x.chunk(world)[rank].clone().requires_grad_()
            out, ln = m(xs)
            xf = x.clone().requires_grad_()
            want = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + m.eps) * g
            if ln.shape != want.shape or not torch.allclose(ln, want, atol=1e-5):
                bad[kind + ":ln"] = tuple(ln.shape)
            # a loss on the gathered output alone, different on every rank: the local rows' gradient is the SUM of
            # all ranks' gradients for them
            w = torch.arange(1, world + 1, dtype=torch.float32)
            (ln.square().sum() * w[rank] + 0.0 * out.sum()).backward()
            (want.square().sum() * w.sum()).backward()
            if not torch.allclose(xs.grad, xf.grad.chunk(world)[rank], rtol=1e-4, atol=1e-5):
                bad[kind + ":dx"] = float((xs.grad - xf.grad.chunk(world)[rank]).abs().max())
        q.put((rank, bad))
    except Exception:  # noqa: BLE001
        import traceback
        q.put((rank, {"exception": traceback.format_exc()[-1500:]}))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def test_return_layernorm_output_gathered():
    """``return_layernorm_output_gathered``: with sequence parallelism the returned normalized output holds all
    rows; its gradient is reduce-scattered back onto the ranks' own rows."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_ln_gathered_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    for rank, bad in res:
        assert not bad, f"rank {rank}: {bad}"
