"""Data-parallel gradient averaging for the flat parameter layout of `FlatMamba`.

The path shards over batch with no data-path collective; the one exchange per step is the average of the
parameter gradients.  One bucket per layer (a contiguous slice of the flat gradient buffer: the layer's 8
tensors with their alignment padding) is all-reduced as soon as the library reports that layer's gradient
kernels enqueued (`pmb_layer_callback`), on a side stream, so the transfer overlaps the remaining
recompute/backward of earlier layers; the embedding bucket goes last (layer index -1).  Works on CPU tensors
with the gloo backend too (no streams), which is how the bucket logic is tested without GPUs.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def layer_bounds(layer_offsets, total):
    """[(start, end)] per layer from the per-layer start offsets and the buffer length; the embedding
    occupies [0, layer_offsets[0])."""
    starts = list(layer_offsets) + [total]
    return [(starts[i], starts[i + 1]) for i in range(len(layer_offsets))]


class GradAllReducer:
    def __init__(self, flat_grads: torch.Tensor, layer_offsets, group=None):
        self.flat = flat_grads
        self.bounds = layer_bounds(layer_offsets, flat_grads.numel())
        self.emb = (0, layer_offsets[0]) if len(layer_offsets) else (0, flat_grads.numel())
        self.group = group
        self.world = dist.get_world_size(group)
        self.cuda = flat_grads.is_cuda
        self.comm = torch.cuda.Stream() if self.cuda else None
        self.pending = []
        self.done_layers = []

    def bucket(self, layer: int) -> torch.Tensor:
        a, b = self.emb if layer < 0 else self.bounds[layer]
        return self.flat[a:b]

    def on_layer_done(self, layer: int, _user=None):
        """Host callback: the gradients of `layer` are complete in stream order on the current stream."""
        self.done_layers.append(layer)
        if self.world == 1:
            return
        t = self.bucket(layer)
        if self.cuda:
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream())
            self.comm.wait_event(ev)
            with torch.cuda.stream(self.comm):
                self.pending.append(dist.all_reduce(t, op=dist.ReduceOp.AVG, group=self.group, async_op=True))
        else:
            self.pending.append((dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.group, async_op=True), t))

    def finish(self):
        """Waits for every bucket; afterwards the current stream sees averaged gradients."""
        for h in self.pending:
            if self.cuda:
                h.wait()
            else:
                work, t = h
                work.wait()
                t.div_(self.world)      # gloo has no AVG
        self.pending.clear()
        if self.cuda:
            torch.cuda.current_stream().wait_stream(self.comm)
        done, self.done_layers = self.done_layers, []
        return done
