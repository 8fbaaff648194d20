"""CUDA-graph capture of modules and of whole training steps (reference: ``pytorch/graph.py:145-1391``).

Two tools:

``capture_step`` / :class:`GraphedStep` records a COMPLETE iteration -- forward under ``autocast``,
backward, gradient collectives and the optimizer step -- into one CUDA graph and replays it.  A
replayed step costs the host one launch, which is what a tensor-parallel step of many small kernels
needs (at TP=8 the per-GPU work of a layer is a few hundred microseconds; the eager launch path is
slower than the GPU).  Everything that varies between steps lives on the device: the optimizer's step
count (``FusedAdam(capturable=True)``), delayed-scaling amax histories and scales, and the call
numbers of the fused collective GEMMs (kept by those kernels themselves).

``make_graphed_callables`` keeps the reference's per-callable interface: each callable gets a
forward graph and a backward graph with static buffers, spliced into autograd.  ``_order`` captures
the graphs of several model chunks and micro-batches in pipeline-schedule order out of one memory
pool; ``cache_quantized_params`` keeps weight quantization out of the forward graphs and refreshes
the cached FP8 weights in place when ``is_first_microbatch`` says the weights changed.

Without CUDA the callables are returned unchanged (eager).
"""
from __future__ import annotations

import warnings
from typing import Callable, Dict, List, Optional, Sequence, Tuple, Union

import torch

from .quantization import DelayedScalingRecipeState, FP8GlobalStateManager, autocast


_IS_GRAPH_CAPTURING = [False]


def set_capture_start() -> None:
    """Mark the beginning of a capture (``make_graphed_callables`` does this itself; frameworks that capture by
    hand call it so that modules can tell, via ``is_graph_capturing``, that host synchronisations are off limits)."""
    _IS_GRAPH_CAPTURING[0] = True


def set_capture_end() -> None:
    _IS_GRAPH_CAPTURING[0] = False


def is_graph_capturing() -> bool:
    return _IS_GRAPH_CAPTURING[0]


def graph_pool_handle():
    """An opaque token naming a CUDA-graph memory pool, to share one pool between several captures."""
    return torch.cuda.graph_pool_handle()


def _tree_tensors(args):
    return tuple(a for a in args if isinstance(a, torch.Tensor))


def _te_modules(fn) -> list:
    from .modules.base import TransformerEngineBaseModule

    if not isinstance(fn, torch.nn.Module):
        return []
    return [m for m in fn.modules() if isinstance(m, TransformerEngineBaseModule)]


# --------------------------------------------------------------------------- whole-step capture
class GraphedStep:
    """One training (or inference) step as a single CUDA graph.

    ``step_fn(*static_inputs)`` must contain the whole iteration: ``zero_grad(set_to_none=True)``,
    forward, ``backward()``, gradient synchronisation, ``optimizer.step()`` (a capturable optimizer), and
    return the tensors the caller wants to read (the loss).  It is run ``warmup`` times eagerly on a side
    stream (allocator, lazily created communication contexts, autotuned state settle), then recorded.
    Calling the object copies new inputs into the static input buffers and replays; the returned
    tensors are the static outputs, overwritten by the next replay.

    ``before_capture`` runs after the warm-up and before the recording (e.g. ``optimizer.zero_grad``).

    ``sync_group``: process group whose ranks replay this graph together.  A one-element all-reduce is
    recorded at the head of the graph so that no rank starts replay ``n + 1`` before every rank has
    finished replay ``n``; the fused collective kernels rely on that when they reuse a communication
    buffer across the replay boundary.
    """

    def __init__(self, step_fn: Callable, static_inputs: Sequence[torch.Tensor] = (), *, warmup: int = 3,
                 sync_group=None, pool=None, before_capture: Optional[Callable] = None):
        from .modules.base import bump_weights_epoch

        assert torch.cuda.is_available(), "GraphedStep needs a CUDA device"
        self.step_fn = step_fn
        self.static_inputs = tuple(static_inputs)
        self.sync_group = sync_group
        self._sync_word = torch.zeros(1, device="cuda") if sync_group is not None else None
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(max(warmup, 1)):
                self._run()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        # memory the warm-up left cached in the ordinary pool cannot serve the graph's private pool: drop
        # what the caller can drop (``before_capture``: typically the warm-up gradients) and release it
        if before_capture is not None:
            before_capture()
        import gc

        gc.collect()
        torch.cuda.empty_cache()
        bump_weights_epoch()  # weight quantization must be part of the recording, not a cache hit
        self.graph = torch.cuda.CUDAGraph()
        self.kernels_per_replay = 0
        from .ops import _ext

        before = _ext.get().launch_count() if _ext.available() else 0
        with torch.cuda.graph(self.graph, pool=pool, capture_error_mode="thread_local"):
            out = self._run()
        self.kernels_per_replay = (_ext.get().launch_count() - before) if _ext.available() else 0
        self._is_tuple = isinstance(out, (tuple, list))
        self.static_outputs = tuple(out) if self._is_tuple else (out,)
        self.replays = 0

    def _run(self):
        if self.sync_group is not None:
            torch.distributed.all_reduce(self._sync_word, group=self.sync_group)
        return self.step_fn(*self.static_inputs)

    def __call__(self, *inputs):
        assert len(inputs) == len(self.static_inputs), "graphed step called with a different number of inputs"
        for dst, src in zip(self.static_inputs, inputs):
            if src is not dst:
                dst.copy_(src, non_blocking=True)
        self.graph.replay()
        self.replays += 1
        return self.static_outputs if self._is_tuple else self.static_outputs[0]

    def release(self) -> None:
        """Drop the recorded graph and its memory pool.  Do this before destroying a process group whose
        collectives were recorded: tearing down a communicator that a live graph still references can block."""
        self.static_outputs = ()
        if self.graph is not None:
            self.graph.reset()
            self.graph = None


def capture_step(step_fn: Callable, static_inputs: Sequence[torch.Tensor] = (), **kw) -> GraphedStep:
    """Record ``step_fn`` (a whole iteration) into one CUDA graph; see :class:`GraphedStep`."""
    return GraphedStep(step_fn, static_inputs, **kw)


# --------------------------------------------------------------------------- per-callable graphs
def _save_delayed_state(mods) -> list:
    """Copies of every delayed-scaling scale / amax history of ``mods`` (warm-up must not advance them)."""
    saved = []
    for m in mods:
        for st in m._states.values():
            if isinstance(st, DelayedScalingRecipeState):
                saved.append((st, st.scale.clone(), st.amax_history.clone()))
    return saved


def _restore_delayed_state(saved) -> None:
    for st, scale, hist in saved:
        st.scale.copy_(scale)
        st.amax_history.copy_(hist)


class _Graphed:
    """Forward and backward graphs of one callable for one set of static buffers."""

    def __init__(self, fn: Callable, sample_args: Tuple, sample_kwargs: Dict, enabled: bool, recipe,
                 amax_reduction_group, cache_quantized_params: bool, allow_unused_input: bool, pool):
        self.fn = fn
        self.enabled, self.recipe, self.group = enabled, recipe, amax_reduction_group
        self.cache_quantized_params = cache_quantized_params
        self.allow_unused = allow_unused_input
        self.pool = pool
        self.te_mods = _te_modules(fn)
        self.params = tuple(p for p in fn.parameters() if p.requires_grad) if isinstance(fn, torch.nn.Module) else ()
        self.static_in = tuple(a.detach().clone().requires_grad_(a.requires_grad) if isinstance(a, torch.Tensor) else a
                               for a in sample_args)
        self.kwargs = dict(sample_kwargs)
        self.fwd_graph = self.bwd_graph = None
        self._seen_epoch = -1

    # ---- pieces used by the capture driver
    def _call(self):
        with autocast(enabled=self.enabled, recipe=self.recipe, amax_reduction_group=self.group, _graph=True):
            return self.fn(*self.static_in, **self.kwargs)

    def _grad_inputs(self):
        return [t for t in _tree_tensors(self.static_in) if t.requires_grad] + list(self.params)

    def warmup(self, n: int) -> None:
        for _ in range(n):
            out = self._call()
            outs = out if isinstance(out, tuple) else (out,)
            need = [o for o in outs if isinstance(o, torch.Tensor) and o.requires_grad]
            if need:
                grads = torch.autograd.grad(need, self._grad_inputs(), [torch.ones_like(o) for o in need],
                                            allow_unused=True)
                del grads
            del out, outs

    def capture_forward(self) -> None:
        from .modules.base import freeze_weight_caches

        old = freeze_weight_caches(self.cache_quantized_params)  # cached weights: no quantize kernels recorded
        try:
            self.fwd_graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.fwd_graph, pool=self.pool):
                out = self._call()
        finally:
            freeze_weight_caches(old)
        self.out_is_tuple = isinstance(out, tuple)
        self.static_out = out if self.out_is_tuple else (out,)
        self.static_gout = tuple(torch.zeros_like(o) if o.requires_grad else None for o in self.static_out)

    def capture_backward(self) -> None:
        self.grad_targets = self._grad_inputs()
        need = [(o, g) for o, g in zip(self.static_out, self.static_gout) if g is not None]
        self.bwd_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.bwd_graph, pool=self.pool):
            self.static_gin = torch.autograd.grad([o for o, _ in need], self.grad_targets, [g for _, g in need],
                                                  allow_unused=True)
        if not self.allow_unused:
            unused = [i for i, g in enumerate(self.static_gin) if g is None]
            if unused:
                raise RuntimeError(f"{len(unused)} inputs / parameters of the graphed callable received no gradient; "
                                   "pass allow_unused_input=True to accept that")

    # ---- replay
    def _refresh_weights(self, is_first_microbatch) -> None:
        if not self.cache_quantized_params:
            return
        from .modules.base import weights_epoch

        changed = self._seen_epoch != weights_epoch()
        if is_first_microbatch is True or (is_first_microbatch is None and changed):
            with autocast(enabled=self.enabled, recipe=self.recipe, _graph=True):
                for m in self.te_mods:
                    m.requantize_cached_weights()
            self._seen_epoch = weights_epoch()

    def __call__(self, *args, is_first_microbatch: Optional[bool] = None, **kwargs):
        graphed = self
        for k, v in kwargs.items():  # tensor keyword arguments are static buffers too
            dst = self.kwargs.get(k)
            if isinstance(dst, torch.Tensor) and isinstance(v, torch.Tensor) and dst.data_ptr() != v.data_ptr():
                dst.copy_(v)
        self._refresh_weights(is_first_microbatch)
        statics = _tree_tensors(self.static_in)
        given = _tree_tensors(args)
        assert len(given) == len(statics), "graphed callable called with a different number of tensors"
        # autograd sees: inputs that do not need grad, then (inputs needing grad + parameters) in the
        # order the captured backward returns their gradients
        ordered = [a for a, s in zip(given, statics) if s.requires_grad] + list(self.params)
        skipped = [a for a, s in zip(given, statics) if not s.requires_grad]

        class _Replay(torch.autograd.Function):
            @staticmethod
            def forward(ctx, n_skipped, *t):  # type: ignore[override]
                ctx.n_skipped = n_skipped
                it_s, it_r = iter(t[:n_skipped]), iter(t[n_skipped:])
                for dst in statics:
                    src = next(it_r) if dst.requires_grad else next(it_s)
                    if dst.data_ptr() != src.data_ptr():
                        dst.copy_(src)
                graphed.fwd_graph.replay()
                return tuple(o.detach() for o in graphed.static_out)

            @staticmethod
            def backward(ctx, *gouts):  # type: ignore[override]
                for dst, src in zip(graphed.static_gout, gouts):
                    if dst is not None and src is not None:
                        dst.copy_(src)
                graphed.bwd_graph.replay()
                grads = tuple(g.detach() if g is not None else None for g in graphed.static_gin)
                return (None,) + (None,) * ctx.n_skipped + grads

        out = _Replay.apply(len(skipped), *skipped, *ordered)
        return out if self.out_is_tuple else out[0]


class _MicrobatchCycle:
    """Callable of one model chunk under a pipeline ``_order``: call ``i`` of an iteration replays the
    graphs of micro-batch ``i`` (each micro-batch has its own static activations, because several are in
    flight between their forward and their backward)."""

    def __init__(self, per_microbatch: List[_Graphed]):
        self.per_microbatch = per_microbatch
        self._next = 0

    def __call__(self, *args, **kwargs):
        g = self.per_microbatch[self._next]
        self._next = (self._next + 1) % len(self.per_microbatch)
        return g(*args, **kwargs)

    def reset(self) -> None:
        self._next = 0


def make_graphed_callables(modules: Union[Callable, Sequence[Callable]], sample_args, num_warmup_iters: int = 3,
                           allow_unused_input: bool = False, sample_kwargs=None, enabled: bool = False,
                           calibrating: bool = False, recipe=None, amax_reduction_group=None,
                           cache_quantized_params: bool = False, pool=None, fp8_enabled: Optional[bool] = None,
                           fp8_recipe=None, fp8_weight_caching: Optional[bool] = None, _order=None,
                           retain_graph_in_backward: bool = False, fp8_calibrating: Optional[bool] = None,
                           fp8_group=None, pre_warmup_hook: Optional[Callable] = None,
                           post_warmup_hook: Optional[Callable] = None, _num_layers_per_chunk=None,
                           _reuse_graph_input_output_buffers: bool = False, clone_param_grads_on_return: bool = False,
                           capture_time_hooks=None):
    """Graph one callable or a tuple of callables (``sample_args`` then holds one tuple per callable).

    ``_order`` (a pipeline schedule such as ``[1, 2, 1, 2, -2, -1, -2, -1]``: ``+c`` = forward of chunk ``c``'s
    next micro-batch, ``-c`` = backward of chunk ``c``'s oldest outstanding micro-batch): ``modules`` holds one
    callable per chunk and ``sample_args`` one entry per (micro-batch, chunk) pair, micro-batch major.  Graphs
    are captured in schedule order from one pool, so a backward frees its activations for the forwards that
    follow it, like the eager schedule.  Returns one callable per chunk.
    """
    if not _IS_GRAPH_CAPTURING[0]:
        set_capture_start()
        try:
            return make_graphed_callables(modules, sample_args, num_warmup_iters, allow_unused_input, sample_kwargs,
                                          enabled, calibrating, recipe, amax_reduction_group, cache_quantized_params,
                                          pool, fp8_enabled, fp8_recipe, fp8_weight_caching, _order,
                                          retain_graph_in_backward, fp8_calibrating=fp8_calibrating,
                                          fp8_group=fp8_group, pre_warmup_hook=pre_warmup_hook,
                                          post_warmup_hook=post_warmup_hook,
                                          _num_layers_per_chunk=_num_layers_per_chunk,
                                          _reuse_graph_input_output_buffers=_reuse_graph_input_output_buffers,
                                          clone_param_grads_on_return=clone_param_grads_on_return,
                                          capture_time_hooks=capture_time_hooks)
        finally:
            set_capture_end()
    if fp8_enabled is not None:
        enabled = fp8_enabled
    if fp8_recipe is not None:
        recipe = fp8_recipe
    if fp8_weight_caching is not None:
        cache_quantized_params = fp8_weight_caching
    if fp8_calibrating is not None:
        calibrating = fp8_calibrating
    if fp8_group is not None:
        amax_reduction_group = fp8_group
    for opt, val in (("_num_layers_per_chunk", _num_layers_per_chunk),
                     ("_reuse_graph_input_output_buffers", _reuse_graph_input_output_buffers),
                     ("clone_param_grads_on_return", clone_param_grads_on_return),
                     ("capture_time_hooks", capture_time_hooks)):
        if val:
            raise NotImplementedError(f"make_graphed_callables({opt}=...) is not implemented")
    if calibrating:
        raise NotImplementedError("calibration runs eagerly: graph the callables after calibrating")
    if retain_graph_in_backward:
        raise NotImplementedError("retain_graph_in_backward is not supported by the captured backward graphs")
    single = not isinstance(modules, (tuple, list))
    mods = (modules,) if single else tuple(modules)
    if not torch.cuda.is_available():
        return modules

    def as_tuple(a):
        return a if isinstance(a, tuple) else (a,)

    pool = pool if pool is not None else torch.cuda.graph_pool_handle()
    if _order is None:
        args = (sample_args,) if single else tuple(sample_args)
        kwargs = ({} if sample_kwargs is None else sample_kwargs,) if single else tuple(sample_kwargs or [{}] * len(mods))
        assert len(args) == len(mods), "one sample_args entry per callable"
        units = [_Graphed(m, as_tuple(a), k, enabled, recipe, amax_reduction_group, cache_quantized_params,
                          allow_unused_input, pool) for m, a, k in zip(mods, args, kwargs)]
        schedule = [("f", u) for u in units] + [("b", u) for u in reversed(units)]
        result: list = units
    else:
        chunks = len(mods)
        assert sorted(set(abs(c) for c in _order)) == list(range(1, chunks + 1)), "_order must name every chunk"
        n_mb = sum(1 for c in _order if c == 1)
        assert all(sum(1 for c in _order if c == k) == n_mb and sum(1 for c in _order if c == -k) == n_mb
                   for k in range(1, chunks + 1)), "_order needs as many forwards as backwards for every chunk"
        flat = list(sample_args)
        assert len(flat) == n_mb * chunks, "sample_args needs one entry per (micro-batch, chunk)"
        kws = list(sample_kwargs) if sample_kwargs is not None else [{}] * len(flat)
        per_chunk = [[_Graphed(mods[c], as_tuple(flat[mb * chunks + c]), kws[mb * chunks + c], enabled, recipe,
                               amax_reduction_group, cache_quantized_params, allow_unused_input, pool)
                      for mb in range(n_mb)] for c in range(chunks)]
        nf, nb = [0] * chunks, [0] * chunks
        schedule = []
        for c in _order:
            k = abs(c) - 1
            if c > 0:
                schedule.append(("f", per_chunk[k][nf[k]]))
                nf[k] += 1
            else:
                assert nb[k] < nf[k], "_order runs a backward before its forward"
                schedule.append(("b", per_chunk[k][nb[k]]))
                nb[k] += 1
        units = [u for row in per_chunk for u in row]
        result = [_MicrobatchCycle(row) for row in per_chunk]

    # warm-up on a side stream; delayed-scaling state is put back afterwards so that the numerics of the
    # first real step do not depend on how many warm-up runs were made
    te_mods = [m for u in units for m in u.te_mods]
    saved = _save_delayed_state(te_mods)
    if pre_warmup_hook is not None:
        pre_warmup_hook()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for u in units:
            u.warmup(num_warmup_iters)
    torch.cuda.current_stream().wait_stream(side)
    if post_warmup_hook is not None:
        post_warmup_hook()
    _restore_delayed_state(saved)
    FP8GlobalStateManager._pending = {"forward": [], "backward": []}
    for kind, u in schedule:
        if kind == "f":
            u.capture_forward()
        else:
            u.capture_backward()
    _restore_delayed_state(saved)
    if single:
        return result[0]
    return tuple(result)
