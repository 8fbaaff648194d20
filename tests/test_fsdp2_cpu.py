"""Quantized parameters under the real FSDP2 (``torch.distributed.fsdp.fully_shard``) over gloo: the shards stay
quantized (FP8 bytes and scales are what the all-gather moves), the tensors' ``fsdp_pre_all_gather`` /
``fsdp_post_all_gather`` hooks run, and the forward / backward results equal the unsharded layer's.
(Test model: the reference's ``tests/pytorch/distributed/test_torch_fsdp2.py``.)"""
import functools
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        from torch.distributed.fsdp import fully_shard

        import transformerengine_b200 as te
        from transformerengine_b200.common import recipe as R
        from transformerengine_b200.tensor.float8 import Float8Tensor
        from transformerengine_b200.tensor.mxfp8 import MXFP8Tensor

        calls = {"pre": 0, "post": 0}

        def counted(fn, key):
            @functools.wraps(fn)           # FSDP2 inspects the hook's signature
            def w(self, *a, **k):
                calls[key] += 1
                return fn(self, *a, **k)
            return w

        for cls in (Float8Tensor, MXFP8Tensor):
            cls.fsdp_pre_all_gather = counted(cls.fsdp_pre_all_gather, "pre")
            cls.fsdp_post_all_gather = counted(cls.fsdp_post_all_gather, "post")
        bad = {}
        for name, rec, cls in (("current", R.Float8CurrentScaling(), Float8Tensor),
                               ("mxfp8", R.MXFP8BlockScaling(), MXFP8Tensor)):
            torch.manual_seed(0)
            with te.quantized_model_init(enabled=True, recipe=rec):
                lin = te.Linear(256, 256, bias=False, params_dtype=torch.float32, device="cpu")
                ref = te.Linear(256, 256, bias=False, params_dtype=torch.float32, device="cpu")
            ref.weight.quantize_(lin.weight.dequantize())
            before = dict(calls)
            fully_shard(lin)
            local = lin.weight._local_tensor
            if not isinstance(local, cls) or tuple(local.shape) != (256 // world, 256):
                bad[f"{name}: shard type"] = f"{type(local).__name__} {tuple(local.shape)}"
            torch.manual_seed(5)
            x = torch.randn(128, 256)
            xa, xb = x.clone().requires_grad_(), x.clone().requires_grad_()
            with te.autocast(enabled=True, recipe=rec):
                y, yr = lin(xa), ref(xb)
            y.square().sum().backward()
            yr.square().sum().backward()
            if calls["pre"] == before["pre"] or calls["post"] == before["post"]:
                bad[f"{name}: hooks"] = str(calls)
            if not torch.allclose(y, yr, rtol=1e-5, atol=1e-5):
                bad[f"{name}: forward"] = float((y - yr).abs().max())
            if not torch.allclose(xa.grad, xb.grad, rtol=1e-4, atol=1e-4):
                bad[f"{name}: dgrad"] = float((xa.grad - xb.grad).abs().max())
            # every rank saw the same batch: FSDP averages the weight gradient over the ranks and keeps the row shard
            g = lin.weight.grad._local_tensor
            want = ref.weight.grad.chunk(world, dim=0)[rank]
            if not torch.allclose(g, want, rtol=1e-4, atol=1e-4):
                bad[f"{name}: wgrad shard"] = float((g - want).abs().max())
        # several optimizer steps: the shards are re-quantized by the optimizer (fp32 master weights), and what the
        # next forward pass sees must be exactly the gathered shards (one scale for per-tensor FP8, fresh bytes for
        # MXFP8), i.e. training makes progress and all ranks hold the same full weight
        from transformerengine_b200.tensor.blockwise import Float8BlockwiseQTensor
        from transformerengine_b200.tensor.nvfp4 import NVFP4Tensor
        for name, rec, cls in (("current", R.Float8CurrentScaling(), Float8Tensor),
                               ("mxfp8", R.MXFP8BlockScaling(), MXFP8Tensor),
                               ("nvfp4", R.NVFP4BlockScaling(), NVFP4Tensor),
                               ("block", R.Float8BlockScaling(), Float8BlockwiseQTensor)):
            torch.manual_seed(0)
            with te.quantized_model_init(enabled=True, recipe=rec):
                lin = te.Linear(256, 256, bias=False, params_dtype=torch.float32, device="cpu")
            fully_shard(lin)
            if not isinstance(lin.weight._local_tensor, cls):
                bad[f"{name}: shard type"] = type(lin.weight._local_tensor).__name__
            opt = te.FusedAdam(lin.parameters(), lr=1e-2, master_weights=True)
            torch.manual_seed(7 + rank)
            x = torch.randn(128, 256)
            seen, losses = [], []
            orig = lin.get_quantized_weight

            def spy(weight, quantizer, **kw):
                seen.append((type(weight), weight.dequantize().clone()))
                return orig(weight, quantizer, **kw)

            lin.get_quantized_weight = spy
            for _ in range(4):
                opt.zero_grad()
                with te.autocast(enabled=True, recipe=rec):
                    loss = lin(x).square().mean()
                loss.backward()
                opt.step()
                losses.append(float(loss.detach()))
            if not all(t is cls for t, _ in seen):
                bad[f"{name}: gathered parameter type"] = str([t.__name__ for t, _ in seen])
            if not losses[-1] < 0.7 * losses[0]:
                bad[f"{name}: no progress over optimizer steps"] = str(losses)
            # the weight of the last forward pass == the shards after the third step, gathered in high precision
            local = lin.weight._local_tensor
            # (roll back one step is not possible; compare the NEXT gather instead)
            with te.autocast(enabled=True, recipe=rec):
                lin(x)
            parts = [torch.empty(256 // world, 256) for _ in range(world)]
            dist.all_gather(parts, local.dequantize().contiguous())
            full = torch.cat(parts)
            if not torch.equal(seen[-1][1], full):
                bad[f"{name}: gathered weight != shards"] = float((seen[-1][1] - full).abs().max())
        q.put((rank, bad, None))
    except Exception:  # noqa: BLE001
        import traceback

        q.put((rank, {}, traceback.format_exc()))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def test_quantized_parameters_under_fully_shard():
    pytest.importorskip("torch.distributed.fsdp")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    for rank, bad, tb in res:
        assert tb is None, tb
        assert not bad, f"rank {rank}: {bad}"
