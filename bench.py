"""Flagship benchmark: one Llama-3-8B-architecture pre-training step (forward, backward,
fused Adam with fp32 master weights) at seq 8192, micro-batch 1, MXFP8 block scaling.

    python bench.py --gpus N --steps K --warmup W [--impl ours|reference] [--config NAME]

N = 1: single GPU.  N = 2, 4: data parallel (one sequence per GPU, gradient
all-reduce).  N = 8: tensor parallel with sequence parallelism, fused collective GEMMs, the
whole step replayed from one CUDA graph.  Launched with ``torch.distributed.run`` for N > 1.
Prints one JSON line from rank 0.  Weights are random N(0, 0.02), token ids uniform over the
vocabulary.

``--config`` selects the other benchmark configurations: ``layer12288`` (one sequence-parallel
TransformerLayer, hidden 12288, forward + backward, TP = N), ``llama70b-nvfp4`` (70B-architecture
layers under NVFP4 with full recompute, TP = N, 5 layers per GPU: 40 at N = 8) and ``mixtral``
(8x7B-architecture MoE, expert parallel over N ranks, 4 layers per GPU below N = 8).
"""
import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")
sys.path.insert(0, ROOT)

SEQ = 8192
METRIC = "tokens_per_second"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    # development knobs; the defaults are the benchmarked configuration
    ap.add_argument("--config", default="llama8b", choices=["llama8b", "layer12288", "llama70b-nvfp4", "mixtral"],
                    help="which benchmark configuration to run (default: the Llama-3-8B-architecture step)")
    ap.add_argument("--layers", type=int, default=0, help="0 = the configuration's layer count")
    ap.add_argument("--seq", type=int, default=0, help="0 = the configuration's sequence length")
    ap.add_argument("--recompute", type=int, default=-1, help="-1 auto, 0 off, 1 per-layer recompute")
    ap.add_argument("--recipe", default="", help="override the configuration's recipe")
    ap.add_argument("--graph", type=int, default=-1, help="-1 auto (whole-step CUDA graph where supported), 0 off, 1 on")
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--profile", default="", help="write a per-kernel device-time table of 2 extra steps (rank 0) here")
    ap.add_argument("--fused-comm", type=int, default=1, help="fuse TP collectives into the GEMM kernels")
    ap.add_argument("--tp", type=int, default=0, help="tensor-parallel size; 0 = 8 at 8 GPUs, else 1")
    ap.add_argument("--param-remainders", type=int, default=0,
                    help="keep the fp32 master weights as bf16 parameter + 16-bit remainder (same values, 15 GB less "
                         "memory; measured 1 % slower per step than plain fp32 masters, so off by default)")
    ap.add_argument("--zero", type=int, default=-1,
                    help="data parallel: shard the optimizer over the ranks (-1: on whenever there is data parallelism)")
    return ap.parse_args()


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU every 200 ms through NVML (read only)."""

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.sm_max = index, [], set(), None
        self._stop_evt = threading.Event()

    def run(self):
        try:
            import pynvml as N
            N.nvmlInit()
            h = N.nvmlDeviceGetHandleByIndex(self.index)
            self.sm_max = N.nvmlDeviceGetMaxClockInfo(h, N.NVML_CLOCK_SM)
            names = {N.nvmlClocksThrottleReasonHwSlowdown: "hw_slowdown",
                     N.nvmlClocksThrottleReasonHwThermalSlowdown: "hw_thermal_slowdown",
                     N.nvmlClocksThrottleReasonSwThermalSlowdown: "sw_thermal_slowdown",
                     N.nvmlClocksThrottleReasonSwPowerCap: "sw_power_cap"}
            while not self._stop_evt.is_set():
                self.samples.append(N.nvmlDeviceGetClockInfo(h, N.NVML_CLOCK_SM))
                r = N.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                for bit, nm in names.items():
                    if r & bit:
                        self.reasons.add(nm)
                time.sleep(0.2)
        except Exception as e:  # noqa: BLE001
            self.reasons.add(f"nvml_unavailable:{type(e).__name__}")

    def stop(self):
        self._stop_evt.set()
        self.join(timeout=2)
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.sm_max, "reasons": sorted(self.reasons)}


def physical_gpu_index(local_rank: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_rank])
        except (ValueError, IndexError):
            return local_rank
    return local_rank


def init_dist(n):
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return rank, local, world


def timed_loop(step_fn, steps, world, sampler_index=None):
    """Barrier + synchronize on both sides, CUDA events around exactly `steps` steps, max over ranks."""
    import torch
    import torch.distributed as dist

    sampler = ClockSampler(sampler_index) if sampler_index is not None else None
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    if sampler:
        sampler.start()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for i in range(steps):
        step_fn(i)
    e.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ms = s.elapsed_time(e)
    clocks = sampler.stop() if sampler else None
    if world > 1:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms, clocks


def build_case(args, rank, world):
    """Model, optimizer and data of the selected benchmark configuration.

    Returns a dict with ``step(tokens) -> loss`` (one full training iteration), the pinned host batches, the
    tokens processed per step over all ranks, FLOPs per token and the description for the JSON line."""
    import torch
    import torch.distributed as dist

    import transformerengine_b200 as te
    from transformerengine_b200.models import llama, mixtral
    from transformerengine_b200.parallel import distributed as D
    from transformerengine_b200.parallel.data_parallel import DataParallelGradSync

    recipes = {"mxfp8": te.recipe.MXFP8BlockScaling, "nvfp4": te.recipe.NVFP4BlockScaling,
               "delayed": te.recipe.DelayedScaling, "current": te.recipe.Float8CurrentScaling,
               "block": te.recipe.Float8BlockScaling, "bf16": None}
    name = args.config
    n_batches = 4

    def want_graph(tp, recipe_name):
        """Whole-step CUDA graph: on by request, by default for tensor-parallel steps (their kernels are too
        short for the eager launch path).  Expert-parallel steps read split sizes on the host and stay eager."""
        if name == "mixtral":
            return False
        return args.graph == 1 or (args.graph < 0 and tp > 1)

    def adam(params, graph):
        # fp32 master weights; --param-remainders 1 stores them as the bf16 parameter plus its 16-bit remainder
        return te.FusedAdam(params, lr=1e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, master_weights=True,
                            capturable=graph, store_param_remainders=bool(args.param_remainders))

    if name in ("llama8b", "llama70b-nvfp4"):
        if name == "llama8b":
            tp = args.tp if args.tp > 0 else (world if world == 8 else 1)
            seq = args.seq or 8192
            cfg = llama.LlamaConfig.llama3_8b(num_layers=args.layers or 32)
            recipe_name = args.recipe or "mxfp8"
            recompute = bool(args.recompute) if args.recompute >= 0 else False
            model_name = "llama3-8b-arch" if cfg.num_layers == 32 else f"llama3-8b-arch-{cfg.num_layers}L"
        else:
            # 70B-architecture layers: 40 layers fill 8 x 180 GB under TP=8; fewer GPUs hold 5 layers per GPU
            tp = args.tp if args.tp > 0 else world
            seq = args.seq or 4096
            cfg = llama.LlamaConfig.llama3_70b(num_layers=args.layers or 5 * world)
            recipe_name = args.recipe or "nvfp4"
            recompute = bool(args.recompute) if args.recompute >= 0 else True
            model_name = f"llama3-70b-arch-{cfg.num_layers}L"
        dp = world // tp
        assert dp == 1 or tp == 1, "this benchmark runs pure DP or pure TP"
        cfg.recompute = recompute
        tp_group = dist.group.WORLD if tp > 1 else None
        # every rank initialises its own shard: different seeds under tensor parallelism
        torch.manual_seed(1000 + (rank if tp > 1 else 0))
        if tp > 1 and args.fused_comm:
            te.initialize_ub(tp_group=tp_group)
        model = llama.LlamaModel(cfg, tp_group=tp_group, sequence_parallel=True)
        if dp > 1:
            for p in model.parameters():
                dist.broadcast(p.data, 0)
        graph = want_graph(tp, recipe_name)
        overlap = os.environ.get("TEB200_DP_OVERLAP", "1") == "1"
        zero = None
        if dp > 1 and args.zero != 0:
            from transformerengine_b200.parallel.data_parallel import ShardedOptimizerDataParallel

            zero = ShardedOptimizerDataParallel(model.parameters(), None, overlap=overlap)
            opt = adam(zero.owned_parameters(), graph)
        else:
            opt = adam(model.parameters(), graph)
        recipe = recipes[recipe_name]() if recipes[recipe_name] is not None else None
        grad_sync = DataParallelGradSync(model.parameters(), None, overlap=overlap) if (dp > 1 and zero is None) else None

        def step(tokens):
            opt.zero_grad(set_to_none=True)
            with te.autocast(enabled=recipe is not None, recipe=recipe):
                loss = model(tokens, labels=tokens)
            loss.backward()
            if tp > 1:
                D.allreduce_sequence_parallel_grads(model, tp_group)   # replicated norm weights see 1/tp of the rows
            if grad_sync is not None:
                grad_sync.finish()
            if zero is not None:
                zero.finish_grads()
            opt.step()
            if zero is not None:
                zero.sync_parameters()
            return loss

        gen = torch.Generator().manual_seed(1234 + rank * (1 if dp > 1 else 0))
        host = [torch.randint(0, cfg.vocab_size, (1, seq), generator=gen).pin_memory() for _ in range(n_batches)]
        return dict(step=step, host=host, tokens_per_step=seq * dp, flops_per_token=cfg.flops_per_token(seq),
                    scaling="weak" if tp == 1 else "strong", sync=world > 1, recipe=recipe_name, graph=graph,
                    before_capture=lambda: opt.zero_grad(set_to_none=True),
                    config={"model": model_name, "global_batch": dp, "seq_len": seq,
                            "parallelism": f"tp{tp}-sp" if tp > 1 else (f"dp{dp}" if dp > 1 else "single"),
                            "recipe": recipe_name,
                            "optimizer": "fused-adam fp32 master" + (" (bf16 parameter + 16-bit remainder)" if args.param_remainders else "")
                            + (" sharded over the ranks" if zero is not None else ""),
                            "fused_comm_gemm": bool(tp > 1 and args.fused_comm), "recompute": recompute})

    if name == "layer12288":
        # one sequence-parallel TransformerLayer, forward + backward (no optimizer: a layer microbenchmark)
        tp = args.tp if args.tp > 0 else world
        seq, mb, H, FFN, NH = args.seq or 2048, 2, 12288, 49152, 96
        recipe_name = args.recipe or "mxfp8"
        tp_group = dist.group.WORLD if tp > 1 else None
        torch.manual_seed(1000 + rank)
        if tp > 1 and args.fused_comm:
            te.initialize_ub(tp_group=tp_group)
        init = lambda t: torch.nn.init.normal_(t, 0.0, 0.02)  # noqa: E731
        layer = te.TransformerLayer(H, FFN, NH, layernorm_epsilon=1e-5, hidden_dropout=0.0, attention_dropout=0.0,
                                    init_method=init, output_layer_init_method=init, self_attn_mask_type="causal",
                                    tp_group=tp_group, tp_size=tp, params_dtype=torch.bfloat16,
                                    sequence_parallel=tp > 1, set_parallel_mode=tp > 1, fuse_qkv_params=True,
                                    activation="gelu", normalization="LayerNorm", device="cuda",
                                    attn_input_format="sbhd")
        recipe = recipes[recipe_name]() if recipes[recipe_name] is not None else None
        gen = torch.Generator().manual_seed(1234)
        host = [torch.randn(seq // tp, mb, H, generator=gen).to(torch.bfloat16).pin_memory() for _ in range(n_batches)]

        def step(x):
            for p in layer.parameters():
                p.grad = None
            x = x.detach().requires_grad_()
            with te.autocast(enabled=recipe is not None, recipe=recipe):
                y = layer(x)
            loss = y.float().square().mean()
            loss.backward()
            return loss

        per_layer = H * 3 * H + H * H + 2 * H * FFN
        return dict(step=step, host=host, tokens_per_step=seq * mb, scaling="strong", sync=world > 1,
                    flops_per_token=6.0 * per_layer + 6.0 * seq * H, recipe=recipe_name,
                    graph=want_graph(tp, recipe_name),
                    config={"model": "transformer-layer-h12288", "global_batch": mb, "seq_len": seq,
                            "parallelism": f"tp{tp}-sp" if tp > 1 else "single", "recipe": recipe_name,
                            "optimizer": "none (forward + backward of one layer)",
                            "fused_comm_gemm": bool(tp > 1 and args.fused_comm), "recompute": False})

    if name == "mixtral":
        # expert parallel over all ranks; attention / router / embeddings are replicated and data parallel.
        # The full 32-layer model holds 46.7 G parameters: 8 ranks fit it, fewer ranks run 4 layers per GPU.
        ep = world
        seq = args.seq or 4096
        layers = args.layers or (32 if world == 8 else 4 * world)
        recipe_name = args.recipe or "mxfp8"
        cfg = mixtral.MixtralConfig.mixtral_8x7b(num_layers=layers)
        ep_group = dist.group.WORLD if ep > 1 else None
        torch.manual_seed(0)
        model = mixtral.MixtralModel(cfg, ep_group=ep_group)
        expert_ids = {id(p) for n, p in model.named_parameters() if ".moe.fc" in n}
        shared = [p for p in model.parameters() if id(p) not in expert_ids]
        if ep > 1:
            for p in shared:
                dist.broadcast(p.data, 0)
        opt = adam(model.parameters(), False)
        recipe = recipes[recipe_name]() if recipes[recipe_name] is not None else None
        grad_sync = DataParallelGradSync(shared, None, average=False) if ep > 1 else None

        def step(tokens):
            opt.zero_grad(set_to_none=True)
            with te.autocast(enabled=recipe is not None, recipe=recipe):
                loss = model(tokens, labels=tokens)
            (loss / ep).backward()     # mean over the ranks' sequences: shared gradients are summed below
            if grad_sync is not None:
                grad_sync.finish()
            opt.step()
            return loss

        gen = torch.Generator().manual_seed(1234 + rank)
        host = [torch.randint(0, cfg.vocab_size, (1, seq), generator=gen).pin_memory() for _ in range(n_batches)]
        h, f = cfg.hidden_size, cfg.ffn_hidden_size
        hd = h // cfg.num_heads
        active = layers * (h * (h + 2 * cfg.num_kv_heads * hd) + h * h + cfg.topk * 3 * h * f + h * cfg.num_experts) \
            + cfg.vocab_size * h
        return dict(step=step, host=host, tokens_per_step=seq * ep, scaling="weak", sync=world > 1,
                    flops_per_token=6.0 * active + 6.0 * layers * seq * h, recipe=recipe_name, graph=False,
                    config={"model": "mixtral-8x7b-arch" if layers == 32 else f"mixtral-8x7b-arch-{layers}L",
                            "global_batch": ep, "seq_len": seq, "parallelism": f"ep{ep}" if ep > 1 else "single",
                            "recipe": recipe_name,
                            "optimizer": "fused-adam fp32 master" + (" (bf16 parameter + 16-bit remainder)" if args.param_remainders else ""),
                            "fused_ep": os.environ.get("TEB200_FUSED_EP", "1") == "1", "recompute": False})
    raise SystemExit(f"unknown --config {name}")


def profile_steps(step_fn, path, rank, world, ms_per_step):
    """Two more steps under torch.profiler (CUDA activity, rank 0): device time per kernel name, NCCL kernels
    included, and the share of the step in which no kernel ran.  Profiled steps are never timed for the result."""
    import torch
    import torch.distributed as dist

    n = 2
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    if rank != 0:
        for i in range(n):
            step_fn(i)
        torch.cuda.synchronize()
        return
    with torch.profiler.profile(activities=[torch.profiler.ProfilerActivity.CUDA]) as prof:
        for i in range(n):
            step_fn(i)
        torch.cuda.synchronize()
    ev = [e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA]
    spans = sorted((e.time_range.start, e.time_range.end) for e in ev)
    busy, cur_s, cur_e = 0.0, None, None
    for s0, e0 in spans:   # union of kernel intervals (kernels on different streams overlap)
        if cur_e is None or s0 > cur_e:
            busy += (cur_e - cur_s) if cur_e is not None else 0.0
            cur_s, cur_e = s0, e0
        else:
            cur_e = max(cur_e, e0)
    busy += (cur_e - cur_s) if cur_e is not None else 0.0
    wall = (spans[-1][1] - spans[0][0]) if spans else 0.0
    table = prof.key_averages().table(sort_by="cuda_time_total", row_limit=45, max_name_column_width=80)
    with open(path, "w") as f:
        f.write(f"steps profiled: {n}; timed (unprofiled) step: {ms_per_step:.2f} ms\n")
        f.write(f"device span of the profiled steps: {wall / 1e3 / n:.2f} ms/step; some kernel running: "
                f"{busy / 1e3 / n:.2f} ms/step; idle: {(wall - busy) / 1e3 / n:.2f} ms/step\n\n")
        f.write(table)


def finish_process_group(world, graphs=()):
    """Leave the job cleanly.  Captured graphs hold NCCL kernels: release them before the communicator goes,
    and never let a stuck teardown keep the process (the result line is already printed)."""
    import threading

    import torch
    import torch.distributed as dist

    for g in graphs:
        g.release()
    torch.cuda.synchronize()
    if world <= 1:
        return
    dist.barrier()
    torch.cuda.synchronize()
    t = threading.Thread(target=dist.destroy_process_group, daemon=True)
    t.start()
    t.join(timeout=20)
    sys.stdout.flush()
    sys.stderr.flush()
    if t.is_alive():
        os._exit(0)


def run_ours(args):
    import torch
    import torch.distributed as dist

    import transformerengine_b200 as te
    from transformerengine_b200.ops import _ext

    rank, local, world = init_dist(args.gpus)
    case = build_case(args, rank, world)
    train_step, host = case["step"], case["host"]
    n_batches = len(host)
    dev = [h.cuda() for h in host]
    # One CUDA graph holds the whole iteration (forward, backward, collectives, optimizer): the host issues
    # one launch per step.
    use_graph = case["graph"]
    C_ = _ext.get()
    if use_graph:
        static_in = torch.empty_like(dev[0])
        static_in.copy_(dev[0])
        try:
            gstep = te.graph.capture_step(train_step, (static_in,), warmup=max(args.warmup, 3),
                                          sync_group=dist.group.WORLD if case["sync"] else None,
                                          before_capture=case.get("before_capture"))
        except Exception as e:  # noqa: BLE001  (the step stays correct without the graph: run it eagerly)
            print(f"[rank {rank}] whole-step capture failed ({type(e).__name__}: {str(e)[:200]}); running eagerly",
                  file=sys.stderr, flush=True)
            torch.cuda.synchronize()
            use_graph = False
    if use_graph:
        per_step = gstep.kernels_per_replay

        def step_device(i):
            gstep(dev[i % n_batches])

        def run_e2e(i):
            return gstep(host[i % n_batches])                     # H2D of this step's inputs from pinned memory
    else:
        per_step = None

        def step_device(i):
            train_step(dev[i % n_batches])

        def run_e2e(i):
            return train_step(host[i % n_batches].cuda(non_blocking=True))

    losses = []

    def step_e2e(i):
        losses.append(float(run_e2e(i).item()))                   # D2H read of the step's result

    for i in range(args.warmup):
        step_device(i)
    torch.cuda.synchronize()
    te.check_status()
    l0 = C_.launch_count()
    ms, clocks = timed_loop(step_device, args.steps, world, physical_gpu_index(local))
    launches = per_step * args.steps if per_step is not None else C_.launch_count() - l0
    te.check_status()
    tokens_per_step = case["tokens_per_step"]
    value = tokens_per_step * args.steps / (ms / 1e3)
    e2e = None
    if not args.skip_e2e:
        step_e2e(0)
        ms2, _ = timed_loop(step_e2e, args.steps, world)
        e2e = {"value": tokens_per_step * args.steps / (ms2 / 1e3), "unit": "tokens/s",
               "h2d_bytes_per_step": host[0].numel() * host[0].element_size(), "d2h_bytes_per_step": 4,
               "ms_per_step": ms2 / args.steps, "last_loss": losses[-1] if losses else None}
    te.check_status()
    if args.profile:
        profile_steps(step_device, args.profile, rank, world, ms / args.steps)
    if rank == 0:
        tflops = value * case["flops_per_token"] / 1e12 / world
        cfg = dict(case["config"])
        cfg["cuda_graph"] = "whole step" if use_graph else "off"
        cfg["l2"] = "inputs and weights far exceed the 126 MB L2"
        out = {"metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
               "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
               "scaling": case["scaling"], "vs_baseline": None, "dtype": "bf16+" + case["recipe"],
               "data": "synthetic", "impl": "ours", "config": cfg,
               "tflops_per_gpu": tflops, "clocks": clocks, "e2e": e2e, "gpu_launches": int(launches),
               "peak_mem_gb": torch.cuda.max_memory_allocated() / 2**30}
        print(json.dumps(out), flush=True)
    finish_process_group(world, [gstep] if use_graph else [])


def run_reference(args):
    """Same step through the unmodified reference installed under baseline/_ref."""
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    try:
        if not os.path.isdir(os.path.join(ref_dir, "transformer_engine")):
            raise ImportError("baseline/_ref holds no transformer_engine install: the offline build of the unmodified "
                              "reference stops in common/fused_attn/*.cu, which need a newer cudnn-frontend than "
                              "the 1.18 headers of this image (no member set_ragged_offset_multiplier)")
        sys.path.insert(0, ref_dir)
        import torch
        import transformer_engine.pytorch as rte
        from transformer_engine.common import recipe as rrecipe
    except Exception as e:  # noqa: BLE001
        print(json.dumps({"impl": "reference", "unavailable": f"{type(e).__name__}: {str(e)[:300]}"}), flush=True)
        return
    import torch.distributed as dist

    rank, local, world = init_dist(args.gpus)
    torch.manual_seed(0)
    tp = args.tp if args.tp > 0 else (world if world == 8 else 1)
    dp = world // tp
    if args.config != "llama8b":
        print(json.dumps({"impl": "reference", "unavailable": "the reference arm covers --config llama8b only"}), flush=True)
        return
    args.layers, args.seq = args.layers or 32, args.seq or SEQ
    V, H, L, NH, NKV, FFN = 128256, 4096, args.layers, 32, 8, 14336
    tp_group = dist.group.WORLD if tp > 1 else None
    init = lambda t: torch.nn.init.normal_(t, 0.0, 0.02)  # noqa: E731

    class RefLlama(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.emb = torch.nn.Embedding(V, H, dtype=torch.bfloat16, device="cuda")
            self.layers = torch.nn.ModuleList([
                rte.TransformerLayer(H, FFN, NH, num_gqa_groups=NKV, layernorm_epsilon=1e-5, hidden_dropout=0.0,
                                     attention_dropout=0.0, init_method=init, output_layer_init_method=init,
                                     layer_number=i + 1, self_attn_mask_type="causal", tp_group=tp_group,
                                     tp_size=tp, params_dtype=torch.bfloat16, sequence_parallel=tp > 1,
                                     set_parallel_mode=tp > 1, fuse_qkv_params=True, bias=False,
                                     activation="swiglu", normalization="RMSNorm", attn_input_format="sbhd")
                for i in range(L)])
            self.norm = rte.RMSNorm(H, eps=1e-5, params_dtype=torch.bfloat16)
            self.head = rte.Linear(H, V, bias=False, init_method=init, params_dtype=torch.bfloat16)
            self.rope = rte.RotaryPositionEmbedding(H // NH, rotary_base=500000.0)

        def forward(self, tokens, recompute):
            x = self.emb(tokens.t().contiguous())
            if tp > 1:
                x = x.chunk(tp, dim=0)[rank].contiguous()
            f = self.rope(tokens.shape[1]).cuda()
            for layer in self.layers:
                if recompute:
                    x = rte.checkpoint(layer, x, rotary_pos_emb=f)
                else:
                    x = layer(x, rotary_pos_emb=f)
            x = self.norm(x)
            if tp > 1:
                xs = [torch.empty_like(x) for _ in range(tp)]
                dist.all_gather(xs, x)
                xs[rank] = x
                x = torch.cat(xs, dim=0)
            logits = self.head(x)
            tgt = torch.full_like(tokens.t(), -100)
            tgt[:-1] = tokens.t()[1:]
            return torch.nn.functional.cross_entropy(logits.reshape(-1, V).float(), tgt.reshape(-1), ignore_index=-100)

    model = RefLlama()
    opt = rte.optimizers.FusedAdam(model.parameters(), lr=1e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1,
                                   master_weights=True)
    rec = rrecipe.MXFP8BlockScaling()
    recompute = bool(args.recompute) if args.recompute >= 0 else False
    gen = torch.Generator().manual_seed(1234 + rank * (1 if dp > 1 else 0))
    host = [torch.randint(0, V, (1, args.seq), generator=gen).pin_memory() for _ in range(4)]
    dev = [h.cuda() for h in host]

    def train_step(tok):
        opt.zero_grad(set_to_none=True)
        with rte.autocast(enabled=True, recipe=rec):
            loss = model(tok, recompute)
        loss.backward()
        if dp > 1:
            for p in model.parameters():
                if p.grad is not None:
                    dist.all_reduce(p.grad)
                    p.grad.div_(dp)
        opt.step()
        return loss

    for i in range(args.warmup):
        train_step(dev[i % 4])
    ms, clocks = timed_loop(lambda i: train_step(dev[i % 4]), args.steps, world, physical_gpu_index(local))
    value = args.seq * dp * args.steps / (ms / 1e3)
    losses = []

    def e2e_step(i):
        losses.append(float(train_step(host[i % 4].cuda(non_blocking=True)).item()))

    e2e_step(0)
    ms2, _ = timed_loop(e2e_step, args.steps, world)
    if rank == 0:
        print(json.dumps({"metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
                          "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
                          "scaling": "weak" if tp == 1 else "strong", "vs_baseline": None, "dtype": "bf16+mxfp8",
                          "data": "synthetic", "impl": "reference",
                          "config": {"model": "llama3-8b-arch", "global_batch": dp, "seq_len": args.seq,
                                     "parallelism": f"tp{tp}-sp" if tp > 1 else (f"dp{dp}" if dp > 1 else "single"),
                                     "recompute": recompute},
                          "clocks": clocks,
                          "e2e": {"value": args.seq * dp * args.steps / (ms2 / 1e3), "unit": "tokens/s",
                                  "h2d_bytes_per_step": host[0].numel() * 8, "d2h_bytes_per_step": 4}}), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    if os.environ.get("TEB200_HANG_DUMP_S"):
        # development aid: print every thread's Python stack and exit if the run takes longer than this
        import faulthandler

        faulthandler.dump_traceback_later(int(os.environ["TEB200_HANG_DUMP_S"]), exit=True)
    a = parse()
    if a.impl == "reference":
        run_reference(a)
    else:
        run_ours(a)
