"""Auxiliary subsystems on CPU: debug features, activation offload, parallel cross entropy,
export mode, utilities."""
import os

import pytest

import torch

import transformerengine_b200 as te
from transformerengine_b200 import debug
from transformerengine_b200.cpu_offload import get_cpu_offload_context
from transformerengine_b200.cross_entropy import parallel_cross_entropy
from transformerengine_b200.debug import debug_api


def test_debug_logging_and_disable(tmp_path):
    torch.manual_seed(0)
    lin = te.Linear(64, 64, bias=False, params_dtype=torch.float32, device="cpu", name="decoder.fc")
    other = te.Linear(64, 64, bias=False, params_dtype=torch.float32, device="cpu", name="decoder.proj")
    x = torch.randn(32, 64)
    debug_api.initialize({
        "stats": {"enabled": True, "layers": {"layer_name_regex_pattern": r".*\.fc$"},
                  "features": {"LogTensorStats": {"tensors": ["activation"], "stats": ["max", "l2_norm"]},
                               "LogFp8TensorStats": {"tensors": ["activation", "weight"], "stats": ["mse"]}}},
        "off": {"enabled": True, "layers": {"layer_names": ["decoder.proj"]},
                "features": {"DisableQuantizationLayer": {}}},
    }, log_dir=str(tmp_path))
    try:
        with te.autocast(enabled=True, recipe=te.recipe.MXFP8BlockScaling()):
            y = lin(x)
            z = other(x)
        recs = debug_api.records()
        stats = {(r["tensor"], r["stat"]) for r in recs}
        assert ("activation", "max") in stats and ("weight", "mse") in stats
        amax = [r["value"] for r in recs if r["stat"] == "max"][0]
        assert abs(amax - x.max().item()) < 1e-6
        # the disabled layer ran in full precision
        assert torch.allclose(z, x @ other.weight.t(), atol=1e-5)
        assert not torch.allclose(y, x @ lin.weight.t(), atol=1e-5)
        debug_api.flush()
        assert os.path.exists(tmp_path / "tensor_stats.jsonl")
    finally:
        debug_api.end_debug()
    assert not debug.is_enabled()


def test_cpu_offload_roundtrip():
    torch.manual_seed(0)
    layers = [torch.nn.Linear(512, 512) for _ in range(3)]
    ctx, sync = get_cpu_offload_context(enabled=True, num_layers=2, model_layers=3)
    x = torch.randn(256, 512, requires_grad=True)
    h = x
    for l in layers:
        with ctx:
            h = torch.tanh(l(h))
        h = sync(h)
    h.sum().backward()
    assert ctx.handler.bytes_offloaded > 0 and not ctx.handler.store
    ref = x.detach().clone().requires_grad_()
    hr = ref
    for l in layers:
        hr = torch.tanh(l(hr))
    hr.sum().backward()
    assert torch.allclose(x.grad, ref.grad, atol=1e-6)


def test_parallel_cross_entropy_single_rank():
    torch.manual_seed(0)
    logits = torch.randn(2, 5, 33, requires_grad=True)
    tgt = torch.randint(0, 33, (2, 5))
    tgt[0, 1] = -100
    loss = parallel_cross_entropy(logits, tgt)
    ref = torch.nn.functional.cross_entropy(logits.reshape(-1, 33), tgt.reshape(-1), reduction="none",
                                            ignore_index=-100).reshape(2, 5)
    assert torch.allclose(loss, ref, atol=1e-5)
    loss.sum().backward()
    g = torch.autograd.grad(ref.sum(), logits)[0]
    assert torch.allclose(logits.grad, g, atol=1e-5)
    red = parallel_cross_entropy(logits.detach(), tgt, reduce_loss=True)
    assert torch.allclose(red, ref.sum() / 9, atol=1e-5)


def test_export_mode_and_utils():
    from transformerengine_b200.export import is_in_onnx_export_mode, onnx_export
    from transformerengine_b200.newton_schulz import newton_schulz
    from transformerengine_b200.utils import DeviceTimers, env_flag, nvtx_range

    assert not is_in_onnx_export_mode()
    with onnx_export(True):
        assert is_in_onnx_export_mode()
    with nvtx_range("x"):
        pass
    t = DeviceTimers()
    with t("a"):
        pass
    assert isinstance(t.summary(), dict)
    assert env_flag("TEB200_SURELY_UNSET", True)
    g = torch.randn(16, 32)
    o = newton_schulz(g, steps=8)
    sv = torch.linalg.svdvals(o.float())
    assert sv.max() < 1.3 and sv.min() > 0.5


def test_quantize_master_weights_single_rank():
    from transformerengine_b200.tensor.utils import quantize_master_weights

    w = torch.nn.Parameter(torch.zeros(8, 4))
    master = torch.arange(16, dtype=torch.float32)
    quantize_master_weights([w], [master], [8])
    assert torch.equal(w.detach().reshape(-1)[8:24], master) and w.detach().reshape(-1)[:8].abs().sum() == 0


def test_debug_per_tensor_scaling_and_fake_quant():
    """PerTensorScaling swaps the recipe's quantizer for FP8 current scaling on the chosen tensors;
    FakeQuant rounds to the low-precision grid and runs the GEMM in high precision."""
    torch.manual_seed(0)
    lin = te.Linear(64, 64, bias=False, params_dtype=torch.float32, device="cpu", name="enc.fc")
    x = torch.randn(32, 64)
    with te.autocast(enabled=True, recipe=te.recipe.MXFP8BlockScaling()):
        base = lin(x)
    debug_api.initialize({"pts": {"enabled": True, "layers": {"layer_names": ["enc.fc"]},
                                  "features": {"PerTensorScaling": {"tensors": ["activation", "weight"], "gemms": ["fprop"]},
                                               "LogFp8TensorStats": {"tensors": ["activation"], "stats": ["mse"]}}}})
    try:
        with te.autocast(enabled=True, recipe=te.recipe.MXFP8BlockScaling()):
            y = lin(x)
        ref = x @ lin.weight.t()
        assert (y - ref).abs().max() < 0.1 * ref.abs().max()
        assert not torch.equal(y, base)  # per-tensor scales round differently from 1x32 block scales
        assert any(r["stat"] == "mse" for r in debug_api.records())
    finally:
        debug_api.end_debug()
    debug_api.initialize({"fq": {"enabled": True, "layers": {"layer_names": ["enc.fc"]},
                                 "features": {"FakeQuant": {"tensors": ["activation"], "gemms": ["fprop"]}}}})
    try:
        with te.autocast(enabled=True, recipe=te.recipe.MXFP8BlockScaling()):
            z = lin(x)
        assert (z - x @ lin.weight.t()).abs().max() < 0.1 * ref.abs().max()
    finally:
        debug_api.end_debug()


def test_torch_compile_wraps_modules_without_changing_results():
    """``torch.compile`` may wrap library modules (quantized autocast included); the kernels stay
    opaque calls and the results equal eager execution."""
    torch.manual_seed(0)
    lin = te.Linear(64, 64, params_dtype=torch.float32, device="cpu")
    x = torch.randn(32, 64)

    def fn(inp):
        with te.autocast(enabled=True, recipe=te.recipe.MXFP8BlockScaling()):
            return lin(inp)

    eager = fn(x)
    compiled = torch.compile(fn, backend="aot_eager")(x)
    torch.testing.assert_close(compiled, eager, rtol=0, atol=0)
    xg = x.clone().requires_grad_()
    torch.compile(fn, backend="aot_eager")(xg).sum().backward()
    assert xg.grad is not None and lin.weight.grad is not None


def test_numerics_debug_counts_saturated_and_flushed_values():
    from transformerengine_b200 import numerics_debug as nd

    x = torch.tensor([0.0, 1e-9, 3.0, 1e6, -1e6])
    q = x.clamp(-448, 448).to(torch.float8_e4m3fn).float()
    assert nd.fp8_tensor_statistics(q, "e4m3") == (2, 2)
    nd.debug(True)
    assert nd.is_debug()
    nd.debug(False)


def test_typed_config_reads_env_once_and_overrides():
    from transformerengine_b200.utils import config as C

    cfg = C.Config.from_env({"TEB200_FUSED_EP": "0", "TEB200_GEMM_BN": "128", "TEB200_ATTN": "library"})
    assert cfg.fused_ep is False and cfg.gemm_tile_n == 128 and cfg.attention_backend == "library"
    assert C.Config.from_env({}).fused_ep is True
    import pytest as _pytest

    with _pytest.raises(ValueError):
        C.Config.from_env({"TEB200_GEMM_BN": "96"})
    with _pytest.raises(ValueError):
        C.Config.from_env({"TEB200_ATTN": "magic"})
    before = C.get_config().fused_context_parallel
    with C.override(fused_context_parallel=not before):
        assert C.get_config().fused_context_parallel is (not before)
    assert C.get_config().fused_context_parallel is before
    text = C.get_config().describe()
    assert "TEB200_FUSED_EP" in text and "NVTE_ALLOW_UNSAFE_PICKLE_EXTRA_STATE" in text


def test_debug_freq_window_struct_yaml_and_nvfp4(tmp_path):
    torch.manual_seed(0)
    cfg_file = tmp_path / "debug.yaml"
    cfg_file.write_text("""
stats:
  enabled: true
  layers:
    layer_name_regex_pattern: "blk\\\\.[0-9]+\\\\.fc"
  features:
    LogTensorStats:
      tensors_struct:
        - tensor: activation
          stats: [mean, std, zeros%]
          freq: 2
        - tensor: weight
          stats: [l2_norm]
          start_step: 1
          end_step: 1
    LogNvfp4TensorStats:
      tensors: [activation]
      stats: [saturated%, mse, scale_inv_max]
""")
    lin = te.Linear(64, 64, bias=False, params_dtype=torch.float32, device="cpu", name="blk.3.fc")
    x = torch.randn(32, 64)
    debug_api.initialize(str(cfg_file), log_dir=str(tmp_path))
    try:
        for _ in range(3):
            with te.autocast(enabled=True, recipe=te.recipe.NVFP4BlockScaling()):
                lin(x)
            debug_api.step()
        recs = debug_api.records()
        by = {}
        for r in recs:
            by.setdefault((r["tensor"], r["stat"]), []).append(r["iteration"])
        assert by[("activation", "mean")] == [0, 2]          # every second iteration
        assert by[("weight", "l2_norm")] == [1]               # only inside its step window
        assert by[("activation", "saturated%")] == [0, 1, 2]
        mean = [r["value"] for r in recs if r["stat"] == "mean"][0]
        std = [r["value"] for r in recs if r["stat"] == "std"][0]
        assert abs(mean - x.mean().item()) < 1e-5 and abs(std - x.std().item()) < 1e-4
        sat = [r["value"] for r in recs if r["stat"] == "saturated%"][0]
        assert 0.0 <= sat <= 100.0
    finally:
        debug_api.end_debug()


def _debug_reduce_worker(rank, world, port, result_q):
    import torch.distributed as dist

    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        torch.manual_seed(0)
        full = torch.randn(64, 64)
        lin = te.Linear(64, 64, bias=False, params_dtype=torch.float32, device="cpu", name="enc.fc")
        debug_api.initialize({"s": {"enabled": True, "layers": {"layer_names": ["enc.fc"]},
                                    "features": {"LogTensorStats": {"tensors": ["activation"],
                                                                    "stats": ["min", "max", "mean", "std", "l2_norm"]}}}})
        debug_api.set_tensor_reduction_group(dist.group.WORLD)
        shard = full.chunk(world, dim=0)[rank].contiguous()      # every rank sees its rows only
        with te.autocast(enabled=True, recipe=te.recipe.MXFP8BlockScaling()):
            lin(shard)
        debug_api.step()
        got = {r["stat"]: r["value"] for r in debug_api.records()}
        want = {"min": full.min().item(), "max": full.max().item(), "mean": full.mean().item(),
                "std": full.std().item(), "l2_norm": full.norm().item()}
        err = max(abs(got[k] - want[k]) for k in want)
        debug_api.end_debug()
        result_q.put((rank, err, None))
    except Exception:  # noqa: BLE001
        import traceback

        result_q.put((rank, None, traceback.format_exc()))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def test_debug_stats_are_reduced_over_the_group():
    import socket

    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_debug_reduce_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=30)
    for rank, err, tb in res:
        assert tb is None, tb
        assert err < 1e-4, (rank, err)


def test_newton_schulz_orthogonalises_and_save_original_input():
    torch.manual_seed(0)
    g = torch.randn(24, 64)
    x = te.newton_schulz(g, steps=8)
    s = torch.linalg.svdvals(x.float())
    assert s.max() < 1.3 and s.min() > 0.5          # singular values pulled towards 1
    xt = te.newton_schulz(g.t().contiguous(), steps=8)
    assert torch.allclose(xt, x.t(), atol=1e-4)
    # save_original_input: same result, the unquantized input is what is kept for the backward
    lin = te.Linear(64, 64, bias=False, params_dtype=torch.float32, device="cpu", save_original_input=True)
    ref = te.Linear(64, 64, bias=False, params_dtype=torch.float32, device="cpu")
    ref.load_state_dict(lin.state_dict())
    inp = torch.randn(32, 64)
    outs = []
    for m in (lin, ref):
        xi = inp.clone().requires_grad_()
        with te.autocast(enabled=True, recipe=te.recipe.MXFP8BlockScaling()):
            y = m(xi)
        y.square().sum().backward()
        outs.append((y.detach(), xi.grad, m.weight.grad))
    for a, b in zip(*outs):
        assert torch.allclose(a, b, atol=1e-6)
    import pytest as _pytest

    with _pytest.raises(NotImplementedError):
        te.Linear(8, 8, device="cpu", symmetric_ar_type="multimem_all_reduce")


def _ns_worker(rank, world, port, result_q):
    import torch.distributed as dist

    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        torch.manual_seed(0)
        full = torch.randn(16, 96)
        want = te.newton_schulz(full, steps=6)
        shard = full.chunk(world, dim=1)[rank].contiguous()
        got = te.newton_schulz(shard, steps=6, group=dist.group.WORLD, partition_dim=1)
        err = (got - want.chunk(world, dim=1)[rank]).abs().max().item()
        # row-sharded tall matrix
        tall = full.t().contiguous()
        got_t = te.newton_schulz(tall.chunk(world, dim=0)[rank].contiguous(), steps=6, group=dist.group.WORLD,
                                 partition_dim=0)
        err = max(err, (got_t - want.t().chunk(world, dim=0)[rank]).abs().max().item())
        result_q.put((rank, err, None))
    except Exception:  # noqa: BLE001
        import traceback

        result_q.put((rank, None, traceback.format_exc()))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def test_newton_schulz_on_a_sharded_matrix():
    import socket

    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_ns_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=30)
    for rank, err, tb in res:
        assert tb is None, tb
        assert err < 1e-4, (rank, err)


def _partial_cast_worker(rank, world, port, result_q):
    import torch.distributed as dist

    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        from transformerengine_b200.tensor import Float8CurrentScalingQuantizer, MXFP8Quantizer
        from transformerengine_b200.tensor.utils import post_all_gather_processing, quantize_master_weights

        torch.manual_seed(0)
        R, C = 64, 96
        master_full = torch.randn(R, C) * 3
        n = R * C
        # uneven split in the middle of a row and of a 32-block
        cut = 37 * C + 50
        lo, hi = (0, cut) if rank == 0 else (cut, n)
        shard = master_full.reshape(-1)[lo:hi].clone()
        errs = {}
        for name, make in (("mxfp8", lambda: MXFP8Quantizer(torch.float8_e4m3fn)),
                           ("fp8cs", lambda: Float8CurrentScalingQuantizer(torch.float8_e4m3fn, device="cpu"))):
            q = make()
            w = q(torch.zeros(R, C))                 # the model weight to refresh (both copies for MXFP8)
            quantize_master_weights([w], [shard], [lo], group=dist.group.WORLD)
            # what a framework does next: every rank contributes the bytes it wrote (sum of disjoint parts)
            def gather(t, mask):
                buf = torch.where(mask, t.view(torch.uint8).reshape(-1), torch.zeros((), dtype=torch.uint8)).int()
                dist.all_reduce(buf)
                t.view(torch.uint8).reshape(-1).copy_(buf.to(torch.uint8))
            flat = torch.arange(n)
            mine = (flat >= lo) & (flat < hi)
            if name == "mxfp8":
                gather(w._rowwise_data, mine)
                mine_t = mine.reshape(R, C).t().contiguous().reshape(-1)
                gather(w._columnwise_data, mine_t)
            else:
                gather(w._data, mine)
            post_all_gather_processing([w])
            ref = make()(master_full)
            if name == "mxfp8":
                ok = torch.equal(w._rowwise_data.view(torch.uint8), ref._rowwise_data.view(torch.uint8)) and \
                    torch.equal(w._columnwise_data.view(torch.uint8), ref._columnwise_data.view(torch.uint8)) and \
                    torch.equal(w._rowwise_scale_inv, ref._rowwise_scale_inv) and \
                    torch.equal(w._columnwise_scale_inv, ref._columnwise_scale_inv)
            else:
                ok = torch.equal(w._data.view(torch.uint8), ref._data.view(torch.uint8)) and \
                    torch.allclose(w._scale_inv.reshape(-1), ref._scale_inv.reshape(-1))
            errs[name] = ok
        result_q.put((rank, errs, None))
    except Exception:  # noqa: BLE001
        import traceback

        result_q.put((rank, None, traceback.format_exc()))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def test_sharded_master_weights_cast_with_partial_amax():
    """Each rank casts only its shard; only amaxes cross the group; the assembled bytes equal a
    quantization of the full master weight."""
    import socket

    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_partial_cast_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=30)
    for rank, errs, tb in res:
        assert tb is None, tb
        assert errs == {"mxfp8": True, "fp8cs": True}, (rank, errs)


def test_helper_ops_cpu_paths():
    """column sums, splits -> offsets, slab re-padding and last-dim padding (the oracle paths of the kernels)."""
    import torch
    from transformerengine_b200 import ops

    x = torch.randn(37, 24)
    torch.testing.assert_close(ops.column_sum(x), x.sum(0))
    s = torch.tensor([3, 0, 5, 2], dtype=torch.int64)
    assert ops.splits_to_offsets(s, multiplier=4).tolist() == [0, 12, 12, 32, 40]
    rows = torch.arange(10 * 8, dtype=torch.float32).reshape(10, 8)
    padded = ops.repad_rows(rows, [3, 0, 5, 2], [4, 0, 8, 4])
    assert padded.shape == (16, 8)
    assert torch.equal(padded[:3], rows[:3]) and padded[3].abs().sum() == 0
    assert torch.equal(padded[4:9], rows[3:8]) and padded[9:12].abs().sum() == 0
    assert torch.equal(ops.repad_rows(padded, [4, 0, 8, 4], [3, 0, 5, 2]), rows)
    p = ops.pad_last_dim(rows, 12)
    assert p.shape == (10, 12) and torch.equal(p[:, :8], rows) and p[:, 8:].abs().sum() == 0
    assert torch.equal(ops.pad_last_dim(p, 8), rows)


@pytest.mark.parametrize("opts", [dict(retain_pinned_cpu_buffers=True), dict(double_buffering=True),
                                  dict(manual_synchronization=True)])
def test_cpu_offload_options(opts):
    """Every option of the offload context changes behaviour, none changes the gradients; two iterations."""
    torch.manual_seed(0)
    layers = [torch.nn.Linear(512, 512) for _ in range(3)]
    res = get_cpu_offload_context(enabled=True, num_layers=2, model_layers=3, **opts)
    ctx, sync = res[0], res[1]
    manual = res[2] if len(res) > 2 else None
    assert (manual is not None) == bool(opts.get("manual_synchronization"))
    for _ in range(2):
        x = torch.randn(256, 512, requires_grad=True)
        h = x
        for i, l in enumerate(layers):
            with ctx:
                h = torch.tanh(l(h))
            h = sync(h)
            if manual is not None:
                manual.start_offload_layer(i)
                manual.release_activation_forward_gpu_memory(i)
        if manual is not None:
            manual.start_reload_layer(1)
        h.sum().backward()
        ref = x.detach().clone().requires_grad_()
        hr = ref
        for l in layers:
            hr = torch.tanh(l(hr))
        hr.sum().backward()
        assert torch.allclose(x.grad, ref.grad, atol=1e-6)
        assert not ctx.handler.store            # everything saved has been handed back
    assert ctx.handler.iteration == 2


def test_cpu_offload_two_forward_passes_in_flight():
    """Entries are keyed by forward pass: a second forward before the first backward does not mix them up."""
    torch.manual_seed(1)
    layers = [torch.nn.Linear(512, 512) for _ in range(2)]
    ctx, sync = get_cpu_offload_context(enabled=True, num_layers=2, model_layers=2)
    outs, xs = [], []
    for _ in range(2):
        x = torch.randn(256, 512, requires_grad=True)
        h = x
        for l in layers:
            with ctx:
                h = torch.tanh(l(h))
            h = sync(h)
        outs.append(h)
        xs.append(x)
    for h, x in zip(outs, xs):
        h.sum().backward()
        ref = x.detach().clone().requires_grad_()
        hr = ref
        for l in layers:
            hr = torch.tanh(l(hr))
        hr.sum().backward()
        assert torch.allclose(x.grad, ref.grad, atol=1e-6)
    assert not ctx.handler.store


def test_grouped_helper_ops_cpu_paths():
    from transformerengine_b200 import ops

    x = torch.randn(12, 16)
    offs = torch.tensor([0, 5, 5, 12], dtype=torch.int32)
    got = ops.grouped_column_sum(x, offs)
    assert torch.allclose(got[0], x[:5].sum(0)) and got[1].abs().sum() == 0 and torch.allclose(got[2], x[5:].sum(0))
    b = torch.randn(3, 16)
    y = ops.grouped_bias_add_(x.clone(), b, offs)
    assert torch.allclose(y[:5], x[:5] + b[0]) and torch.allclose(y[5:], x[5:] + b[2])
    assert torch.allclose(ops.row_dot(x, y), (x * y).sum(-1))


def test_canary_guard_bands_catch_out_of_bounds_writes():
    from transformerengine_b200.utils.canary import GuardedAllocation

    g = GuardedAllocation(guard_bytes=256)
    a = g.empty((4, 8), torch.float32, device="cpu", name="a")
    b = g.empty((3,), torch.uint8, device="cpu", name="b")
    a.normal_()
    b.zero_()
    g.check()                                        # writes inside the tensors are fine
    raw_b = g._allocs[1][1]
    raw_b[256 + 3] = 0                               # one byte past the end of b (inside its alignment padding)
    bad = g.violations()
    assert len(bad) == 1 and bad[0].startswith("b: byte 3")
    with pytest.raises(AssertionError):
        g.check()


def test_canary_intercepts_wrapper_allocations():
    from transformerengine_b200.utils.canary import GuardedAllocation

    g = GuardedAllocation(guard_bytes=256)
    with g.intercept(device_type="cpu"):
        a = torch.empty(5, 7, dtype=torch.float32, device="cpu")
        z = torch.zeros((3, 2), dtype=torch.int32, device="cpu")
        plain = torch.empty(4)                       # no device named: passes through
    assert len(g._allocs) == 2 and a.shape == (5, 7) and z.abs().sum() == 0 and plain.shape == (4,)
    a.fill_(1.0)
    g.check()
    assert torch.empty(2, device="cpu").shape == (2,)   # restored


def test_reference_module_names_resolve_and_work():
    """``distributed``, ``jit``, ``cpp_extensions``, ``fp8``, ``module`` ... exist under the reference's names."""
    import importlib

    for m in ("distributed", "jit", "cpp_extensions", "fp8", "float8_tensor", "quantized_tensor", "permutation",
              "router", "ep", "module", "constants", "custom_recipes", "numerics_debug", "compile_ops"):
        importlib.import_module("transformerengine_b200." + m)
    from transformerengine_b200 import cpp_extensions as ce, distributed as D, jit

    x, b = torch.randn(4, 8, requires_grad=True), torch.randn(8)
    ref = torch.nn.functional.gelu(x + b, approximate="tanh")
    assert torch.allclose(jit.bias_gelu_fused(x, b), ref, atol=1e-6)
    dx, db = jit.bgrad_dgelu_fused(torch.ones(4, 8), x.detach(), b)
    (gx,) = torch.autograd.grad(ref.sum(), x)
    assert torch.allclose(dx, gx, atol=1e-6) and torch.allclose(db, gx.sum(0), atol=1e-5)
    r = torch.randn(4, 8)
    assert torch.allclose(jit.bias_dropout_add_fused_inference(x.detach(), b, r, 0.1), r + x.detach() + b)
    # grouped GEMM, list form: out[i] = B[i] @ A[i]^T
    A = [torch.randn(6, 8), torch.randn(6, 8)]
    B = [torch.randn(3, 8), torch.randn(5, 8)]
    out = [torch.empty(8, 6)]
    ce.general_grouped_gemm(A, B, out, out_dtype=torch.float32, m_splits=[3, 5], single_output=True)
    assert torch.allclose(out[0][:3], B[0] @ A[0].t(), atol=1e-5) and torch.allclose(out[0][3:], B[1] @ A[1].t(), atol=1e-5)
    assert D.get_distributed_world_size(None) == 1 and D.split_tensor_into_1d_equal_chunks(r, None).numel() == 32
    assert not D.is_fp8_activation_recompute_enabled() and not D.in_fp8_activation_recompute_phase()


def test_quickstart_example_runs_and_learns():
    import importlib.util
    import os as _os

    path = _os.path.join(_os.path.dirname(_os.path.dirname(_os.path.abspath(__file__))), "examples", "quickstart.py")
    spec = importlib.util.spec_from_file_location("quickstart_example", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    losses = mod.main(["--recipe", "mxfp8", "--steps", "6", "--hidden", "256", "--seq", "64"])
    assert losses[-1] < losses[0]


def test_newton_schulz_schedules_and_context_form():
    import os as _os
    import torch.distributed as _dist
    from transformerengine_b200.newton_schulz import (CusolverMpCtx, get_coefficient_iterator, get_coefficients,
                                                      newton_schulz)
    assert get_coefficients(7, "simple") == [(3.4445, -4.7750, 2.0315)] * 7
    q = get_coefficients(7, "quintic")
    assert q[5] == q[0] and len(q) == 7                                   # cycles
    pe = get_coefficients(10, "polar_express")
    assert pe[8] == pe[9] == (1.875, -1.25, 0.375) and abs(pe[0][0] - 8.2051) < 1e-4   # last one repeats
    assert list(get_coefficient_iterator(3, [(1, 2, 3)], "repeat_last")) == [(1, 2, 3)] * 3
    with pytest.raises(ValueError):
        get_coefficients(3, "unknown")
    torch.manual_seed(0)
    g = torch.randn(48, 96)
    # the tuned schedules push the singular values into a band around 1 (they do not converge to exactly 1)
    for kind, lo, hi in (("quintic", 0.6, 1.25), ("polar_express", 0.9, 1.1)):
        o = newton_schulz(g, 8, get_coefficients(8, kind), compute_dtype=torch.float32)
        sv = torch.linalg.svdvals(o.float())
        assert lo < float(sv.min()) and float(sv.max()) < hi, (kind, float(sv.min()), float(sv.max()))
    with pytest.raises(ValueError):
        newton_schulz(g, 4, get_coefficients(3))
    # reference call form: context, in place, nothing returned (single-rank group)
    if not _dist.is_initialized():
        _os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        _os.environ.setdefault("MASTER_PORT", "29533")
        _dist.init_process_group("gloo", rank=0, world_size=1)
        made = True
    else:
        made = False
    try:
        ctx = CusolverMpCtx(_dist.group.WORLD)
        x = g.clone()
        want = newton_schulz(g, 5, get_coefficients(5))
        assert newton_schulz(x, ctx, 5) is None
        torch.testing.assert_close(x, want)
        y = g.clone()
        newton_schulz(y, ctx, num_iterations=6, coefficients=get_coefficients(6, "polar_express"))
        torch.testing.assert_close(y, newton_schulz(g, 6, get_coefficients(6, "polar_express")))
        ctx.destroy()
        with pytest.raises(RuntimeError):
            newton_schulz(x, ctx, 5)
    finally:
        if made:
            _dist.destroy_process_group()


def _ce_worker(rank, world, port, result_q):
    import torch.distributed as dist

    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        torch.manual_seed(0)
        full = torch.randn(12, 64)
        tgt = torch.randint(0, 64, (12,))
        tgt[3] = -100
        errs = []
        for eps in (0.0, 0.2):
            xf = full.clone().requires_grad_()
            want = torch.nn.functional.cross_entropy(xf, tgt, label_smoothing=eps, reduction="none")
            want.sum().backward()
            xs = full.chunk(world, dim=1)[rank].clone().requires_grad_()
            got = parallel_cross_entropy(xs, tgt, eps, False, dist.group.WORLD)
            got.sum().backward()
            errs.append(float((got - want).abs().max()))
            errs.append(float((xs.grad - xf.grad.chunk(world, dim=1)[rank]).abs().max()))
        result_q.put((rank, max(errs), None))
    except Exception:  # noqa: BLE001
        import traceback

        result_q.put((rank, None, traceback.format_exc()))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def test_parallel_cross_entropy_label_smoothing_single_rank_and_vocab_sharded():
    import socket

    import torch.multiprocessing as mp

    torch.manual_seed(0)
    x = torch.randn(4, 6, 50, requires_grad=True)
    x2 = x.detach().clone().requires_grad_()
    t = torch.randint(0, 50, (4, 6))
    t[0, 2] = -100
    for reduce in (False, True):
        a = parallel_cross_entropy(x, t, 0.1, reduce)
        b = torch.nn.functional.cross_entropy(x2.reshape(-1, 50), t.reshape(-1), label_smoothing=0.1,
                                              reduction="mean" if reduce else "none")
        torch.testing.assert_close(a.reshape(-1), b.reshape(-1))
        x.grad = x2.grad = None
        a.sum().backward()
        b.sum().backward()
        torch.testing.assert_close(x.grad, x2.grad)
    torch.testing.assert_close(parallel_cross_entropy(None, t, _input=x.detach()), parallel_cross_entropy(x.detach(), t))
    with pytest.raises(ValueError):
        parallel_cross_entropy(x, t, 1.5)
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_ce_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    for rank, err, tb in res:
        assert tb is None, tb
        assert err < 1e-5, (rank, err)


def test_distributed_module_helpers():
    from transformerengine_b200 import distributed as D
    from transformerengine_b200.common import recipe as R
    tracker = D.CudaRNGStatesTracker()
    tracker.add("model-parallel-rng", 4321)
    assert "model-parallel-rng" in D.get_all_rng_states()
    before = D.get_all_rng_states()["model-parallel-rng"].clone()
    w = torch.empty(8, 8)
    D.initialize_affine_weight_gpu(w, lambda t: torch.nn.init.normal_(t), lambda: tracker, partition_dim=1, stride=1)
    assert w.tensor_model_parallel and w.partition_dim == 1
    assert not torch.equal(D.get_all_rng_states()["model-parallel-rng"], before)        # the fork advanced the stream
    saved = dict(D.get_all_rng_states())
    D.set_all_rng_states({})
    assert D.get_all_rng_states() == {}
    D.set_all_rng_states(saved)
    assert isinstance(D.graph_safe_rng_available(), bool) and not D.is_graph_safe_rng_state(torch.zeros(1))
    assert D.has_te_modules(te.Linear(8, 8, device="cpu")) and not D.has_te_modules(torch.nn.Linear(8, 8))
    assert D.has_te_modules(lambda x: x) and te.TransformerLayer in D.get_te_classes()
    # a hand-written checkpoint of a delayed-scaling layer: the two contexts mark the two passes, and the recompute
    # reproduces the first forward although the amax history moved in between
    lin = te.Linear(32, 32, bias=False, params_dtype=torch.float32, device="cpu")
    rec = R.DelayedScaling(amax_history_len=2)
    x = torch.randn(16, 32)
    with te.autocast(enabled=True, recipe=rec):
        lin(x * 5)                                   # fills the history
    fwd_ctx, re_ctx = D.get_activation_recompute_contexts()
    with te.autocast(enabled=True, recipe=rec):
        with fwd_ctx, torch.no_grad():
            assert D.is_fp8_activation_recompute_enabled() and not D.in_fp8_activation_recompute_phase()
            y1 = lin(x)
    with te.autocast(enabled=True, recipe=rec):
        lin(x * 0.01)                                # scales change
    with te.autocast(enabled=True, recipe=rec):
        with re_ctx:
            assert D.in_fp8_activation_recompute_phase()
            y2 = lin(x)
    assert not D.in_fp8_activation_recompute_phase() and not D.is_fp8_activation_recompute_enabled()
    assert torch.equal(y1, y2)
    te.checkpoint(lambda t: t * 2, torch.ones(2, requires_grad=True), use_reentrant=False)
    assert not D.use_reentrant_activation_recompute()
    te.checkpoint(lambda t: t * 2, torch.ones(2, requires_grad=True))
    assert D.use_reentrant_activation_recompute()


def test_offload_graph_and_tensor_util_helpers():
    from transformerengine_b200 import cpu_offload as CO
    from transformerengine_b200 import graph as G
    from transformerengine_b200.tensor import utils as TU
    from transformerengine_b200.tensor.float8 import Float8CurrentScalingQuantizer
    assert not CO.is_cpu_offload_enabled()
    ctx, sync = CO.get_cpu_offload_context(enabled=True, num_layers=1, model_layers=2)
    lin = torch.nn.Linear(512, 512)
    x = torch.randn(256, 512, requires_grad=True)
    with ctx:
        assert CO.is_cpu_offload_enabled()
        keep = torch.tanh(x)
        CO.mark_not_offload(keep)
        CO.mark_activation_offload(keep)            # back to a candidate
        CO.start_offload(keep)
        y = lin(keep).square()
    assert not CO.is_cpu_offload_enabled()
    sync(y).sum().backward()
    assert x.grad is not None and ctx.handler.bytes_offloaded > 0
    assert not G.is_graph_capturing()
    G.set_capture_start()
    assert G.is_graph_capturing()
    G.set_capture_end()
    q = Float8CurrentScalingQuantizer(torch.float8_e4m3fn)(torch.randn(32, 32))
    assert q._transpose is not None
    TU.clear_columnwise_cache(q)
    assert q._transpose is None and q._data is not None
    assert not TU.is_custom(q) and not TU.is_custom(torch.zeros(1)) and not TU.is_custom(None)
    assert TU.cast_master_weights_to_fp8 is TU.quantize_master_weights


def test_utils_helpers():
    from transformerengine_b200 import utils as U
    w = torch.empty(256, 256)
    U.init_method_normal(0.5)(w)
    assert 0.45 < float(w.std()) < 0.55
    U.scaled_init_method_normal(0.5, 8)(w)
    assert 0.11 < float(w.std()) < 0.14                       # 0.5 / sqrt(16)
    U.init_method_constant(2.0)(w)
    assert float(w.min()) == 2.0
    U.get_default_init_method()(w)
    assert 0.02 < float(w.std()) < 0.026
    assert U.divide(12, 4) == 3 and U.ceil_div(7, 2) == 4 and U.round_up_to_nearest_multiple(70, 32) == 96
    with pytest.raises(ValueError):
        U.divide(10, 3)
    a = torch.randn(4, 6, requires_grad=True)
    parts = U.SplitAlongDim.apply(a, 1, 2)
    assert len(parts) == 3
    (parts[0].sum() + 2 * parts[2].sum()).backward()
    assert torch.equal(a.grad, torch.tensor([1.0, 1, 0, 0, 2, 2]).expand(4, 6))
    assert U.combine_tensors([torch.ones(2, 3), torch.zeros(2, 3)], 1).shape == (2, 2, 3)
    assert [p.shape for p in U.split_tensor_along_dim(torch.zeros(4, 6), 1, 3, True)] == [(4, 2)] * 3
    assert U.requires_grad(None, a) and not U.requires_grad(torch.zeros(1))
    assert U.cast_if_needed(a.detach(), torch.bfloat16).dtype == torch.bfloat16 and U.cast_if_needed(None, torch.float32) is None
    t = torch.zeros(10)
    U.clear_tensor_data(t)
    assert t.numel() == 0
    assert U.check_dim_for_fp8_exec(torch.zeros(8, 16)) and not U.check_dim_for_fp8_exec(torch.zeros(8, 8))
    with pytest.raises(ValueError):
        U.assert_dim_for_fp8_exec(torch.zeros(3, 16))
    assert U.needs_quantized_gemm(te.tensor.MXFP8Quantizer()(torch.randn(32, 32))) and not U.needs_quantized_gemm(t)
    U.validate_rng_states_func(lambda: te.CudaRNGStatesTracker())
    with pytest.raises(TypeError):
        U.validate_rng_states_func(lambda: object())
    with pytest.raises(AssertionError):
        U.assert_viewless_tensor(torch.zeros(4)[1:])
    assert U.get_cached_ones_tensor(4, torch.float32, "cpu") is U.get_cached_ones_tensor(4, torch.float32, "cpu")
    assert U.devices_match("cpu", torch.device("cpu")) and U.canonicalize_dtype(None) == torch.get_default_dtype()
    assert U.attention_mask_func(torch.zeros(2), torch.tensor([True, False])).tolist() == [-10000.0, 0.0]
    with U.get_nvtx_range_context("x"):
        pass
    assert U.all_close(torch.ones(2), torch.ones(2))


def test_code_written_for_the_reference_runs_after_installing_the_alias():
    """In a fresh interpreter: after ``install_as_transformer_engine()`` the reference's import lines resolve to
    this package's modules (same objects), and a small training step written against them runs."""
    import subprocess
    import sys
    code = r'''
import transformerengine_b200.compat as compat
compat.install_as_transformer_engine()
import torch
import transformer_engine
import transformer_engine.pytorch as te
from transformer_engine.common.recipe import DelayedScaling, Format
from transformer_engine.common import recipe
from transformer_engine.pytorch.distributed import checkpoint, CudaRNGStatesTracker
from transformer_engine.pytorch.module.linear import Linear
from transformer_engine.pytorch.tensor.float8_tensor import Float8Tensor
from transformer_engine.pytorch.optimizers import FusedAdam
from transformer_engine.pytorch.attention.inference import InferenceParams
from transformer_engine.pytorch.attention.dot_product_attention.utils import get_attention_backend
import transformer_engine.pytorch.ops as te_ops
import transformerengine_b200 as ours
assert te is ours and Linear is ours.Linear and recipe.DelayedScaling is DelayedScaling
assert te_ops.Sequential is ours.fusible.Sequential and callable(get_attention_backend)
assert te.Float8Tensor is Float8Tensor
layer = te.TransformerLayer(64, 128, 4, hidden_dropout=0.0, attention_dropout=0.0, params_dtype=torch.float32, device="cpu")
opt = FusedAdam(layer.parameters(), lr=1e-3)
x = torch.randn(8, 2, 64, requires_grad=True)
with te.fp8_autocast(enabled=True, fp8_recipe=DelayedScaling(fp8_format=Format.HYBRID, amax_history_len=4)):
    y = checkpoint(layer, x)
y.square().mean().backward()
opt.step()
try:
    import transformer_engine_torch
    raise SystemExit("the compiled extension of the reference must not resolve")
except ImportError:
    pass
print("ALIAS-OK")
'''
    res = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300,
                         cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    assert res.returncode == 0 and "ALIAS-OK" in res.stdout, res.stdout[-1500:] + res.stderr[-3000:]


def test_multi_tensor_ops_in_the_applier_convention():
    from transformerengine_b200.optimizers import (MultiTensorApply, multi_tensor_applier, multi_tensor_l2norm,
                                                   multi_tensor_scale, multi_tensor_scale_tensor,
                                                   multi_tensor_unscale_l2norm)
    torch.manual_seed(0)
    grads = [torch.randn(5, 7), torch.randn(3), torch.randn(2, 2, 2)]
    flag = torch.zeros(1, dtype=torch.int32)
    total, each = multi_tensor_applier(multi_tensor_l2norm, flag, [grads], True)
    want = torch.stack([g.norm() for g in grads])
    torch.testing.assert_close(each, want)
    torch.testing.assert_close(total, want.square().sum().sqrt().reshape(1))
    total2, each2 = MultiTensorApply(2048 * 32)(multi_tensor_l2norm, flag, [grads], False)
    assert each2.numel() == 0 and torch.equal(total2, total)
    t3, _ = multi_tensor_applier(multi_tensor_unscale_l2norm, flag, [grads], torch.tensor(0.5), False)
    torch.testing.assert_close(t3, total * 0.5)
    out = [torch.empty_like(g) for g in grads]
    multi_tensor_applier(multi_tensor_scale, flag, [grads, out], 0.25)
    assert all(torch.allclose(o, g * 0.25) for o, g in zip(out, grads)) and int(flag) == 0
    multi_tensor_applier(multi_tensor_scale_tensor, flag, [grads, out], torch.tensor(2.0))
    assert all(torch.allclose(o, g * 2) for o, g in zip(out, grads))
    bad = [torch.tensor([1.0, float("inf")])]
    multi_tensor_applier(multi_tensor_scale, flag, [bad, [torch.empty(2)]], 1.0)
    assert int(flag) == 1
