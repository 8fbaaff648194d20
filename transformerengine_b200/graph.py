"""CUDA-graph capture of modules that run under ``autocast`` (reference: ``pytorch/graph.py:145,
1286,1336``).

``make_graphed_callables`` warms a callable up, captures its forward and backward into CUDA
graphs with static input/output buffers, and returns a callable whose every call replays them.
Quantization state is handled the way the modules need it under capture: delayed-scaling
amax/scale updates happen inside the captured region on device tensors, and weight
re-quantization is controlled by a device flag instead of a host branch.

Without CUDA the callables are returned unchanged (eager).
"""
from __future__ import annotations

from typing import Callable, Dict, Optional, Sequence, Tuple, Union

import torch

from .quantization import FP8GlobalStateManager, autocast


def _tree_tensors(args):
    return tuple(a for a in args if isinstance(a, torch.Tensor))


class _Graphed:
    def __init__(self, fn: Callable, sample_args: Tuple, sample_kwargs: Dict, num_warmup: int, enabled: bool, recipe,
                 cache_quantized_params: bool, pool=None):
        self.fn = fn
        self.enabled, self.recipe = enabled, recipe
        self.params = tuple(p for p in fn.parameters() if p.requires_grad) if isinstance(fn, torch.nn.Module) else ()
        self.static_in = tuple(a.detach().clone().requires_grad_(a.requires_grad) if isinstance(a, torch.Tensor) else a
                               for a in sample_args)
        self.kwargs = sample_kwargs
        stream = torch.cuda.Stream()
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            for _ in range(num_warmup):
                out = self._call()
                outs = out if isinstance(out, tuple) else (out,)
                grads = torch.autograd.grad([o for o in outs if o.requires_grad],
                                            [t for t in _tree_tensors(self.static_in) if t.requires_grad] + list(self.params),
                                            [torch.ones_like(o) for o in outs if o.requires_grad], allow_unused=True)
                del out, outs, grads
        torch.cuda.current_stream().wait_stream(stream)
        self.fwd_graph, self.bwd_graph = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
        self.pool = pool if pool is not None else torch.cuda.graph_pool_handle()
        with torch.cuda.graph(self.fwd_graph, pool=self.pool):
            out = self._call()
        self.static_out = out if isinstance(out, tuple) else (out,)
        self.out_is_tuple = isinstance(out, tuple)
        self.static_gout = tuple(torch.zeros_like(o) for o in self.static_out)
        self.grad_targets = [t for t in _tree_tensors(self.static_in) if t.requires_grad] + list(self.params)
        with torch.cuda.graph(self.bwd_graph, pool=self.pool):
            self.static_gin = torch.autograd.grad([o for o in self.static_out if o.requires_grad], self.grad_targets,
                                                  [g for o, g in zip(self.static_out, self.static_gout) if o.requires_grad],
                                                  allow_unused=True)

    def _call(self):
        with autocast(enabled=self.enabled, recipe=self.recipe, _graph=True):
            return self.fn(*self.static_in, **self.kwargs)

    def __call__(self, *args, **kwargs):
        graphed = self
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
                    if src is not None:
                        dst.copy_(src)
                graphed.bwd_graph.replay()
                grads = tuple(g.detach() if g is not None else None for g in graphed.static_gin)
                return (None,) + (None,) * ctx.n_skipped + grads

        out = _Replay.apply(len(skipped), *skipped, *ordered)
        return out if self.out_is_tuple else out[0]


def make_graphed_callables(modules: Union[Callable, Sequence[Callable]], sample_args, num_warmup_iters: int = 3,
                           allow_unused_input: bool = False, sample_kwargs=None, enabled: bool = False,
                           calibrating: bool = False, recipe=None, amax_reduction_group=None,
                           cache_quantized_params: bool = False, pool=None, fp8_enabled: Optional[bool] = None,
                           fp8_recipe=None, fp8_weight_caching: Optional[bool] = None, _order=None):
    """Graph one callable or a tuple of callables (``sample_args`` then holds one tuple per callable)."""
    if fp8_enabled is not None:
        enabled = fp8_enabled
    if fp8_recipe is not None:
        recipe = fp8_recipe
    if fp8_weight_caching is not None:
        cache_quantized_params = fp8_weight_caching
    single = not isinstance(modules, (tuple, list))
    mods = (modules,) if single else tuple(modules)
    args = (sample_args,) if single else tuple(sample_args)
    kwargs = ({} if sample_kwargs is None else sample_kwargs,) if single else tuple(sample_kwargs or [{}] * len(mods))
    if not torch.cuda.is_available():
        return modules
    pool = pool if pool is not None else torch.cuda.graph_pool_handle()
    graphed = tuple(_Graphed(m, a if isinstance(a, tuple) else (a,), k, num_warmup_iters, enabled, recipe,
                             cache_quantized_params, pool) for m, a, k in zip(mods, args, kwargs))
    return graphed[0] if single else graphed
