"""CUDA-graph replay for any inference callable built on these kernels (counterpart of fastbb/graphs.py:34-65).

    from fastbb_b200.graphs import graphed
    f = graphed(model)          # f(x) == model(x), replayed from one graph per input signature

One graph per (shape, dtype, device, stride) signature of the positional tensor arguments, captured on first use after
one warm-up call on a side stream; at most `max_graphs` signatures are kept (their static buffers hold memory).
Outputs are cloned out of the graph's static buffers unless noclone=True. Not for callables with data-dependent
control flow or host synchronisation. The kernels of this package are capture-safe: they take the stream as an
argument, never synchronise, and allocate nothing. The attention kernel's scratch memory belongs to the Graphed object
(attention.Workspaces): the warm-up call creates and zeroes it outside the capture, the captured graphs bake its address
in, and no other Graphed or model shares it.
"""
import torch

from .attention import Workspaces, use_workspaces


def _map_tensors(o, fn):
    if torch.is_tensor(o):
        return fn(o)
    if isinstance(o, (list, tuple)):
        return type(o)(_map_tensors(v, fn) for v in o)
    if isinstance(o, dict):
        return {k: _map_tensors(v, fn) for k, v in o.items()}
    return o


class Graphed:
    def __init__(self, fn, noclone=False, max_graphs=16):
        self.fn, self.noclone, self.max_graphs = fn, noclone, max_graphs
        self._entries, self._pool = {}, None
        self._workspaces = Workspaces()

    def _capture(self, xs):
        static_in = [x.clone() for x in xs]
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side), use_workspaces(self._workspaces):
            self.fn(*static_in)
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, pool=self._pool), use_workspaces(self._workspaces):
            static_out = self.fn(*static_in)
        self._pool = graph.pool()
        return graph, static_in, static_out

    def __call__(self, *xs):
        key = tuple((tuple(x.shape), x.dtype, x.device, x.stride()) for x in xs)
        entry = self._entries.get(key)
        if entry is None:
            if len(self._entries) >= self.max_graphs:
                self._entries.clear()
                self._pool = None
            entry = self._entries[key] = self._capture(xs)
        graph, static_in, static_out = entry
        for dst, src in zip(static_in, xs):
            dst.copy_(src)
        graph.replay()
        return static_out if self.noclone else _map_tensors(static_out, torch.clone)


def graphed(fn, noclone=False, max_graphs=16):
    return Graphed(fn, noclone, max_graphs)
