"""Host-to-host inference with the PCIe copies hidden behind compute.

A forward pass of the headline workload moves 14 MB to the device and 50 MB of features back; done on the compute stream
that is about a millisecond in which the SMs idle. HostPipeline keeps `depth` device input buffers and pinned host
output buffers, copies on two side streams (host->device, device->host) and chains the three streams with events, so
that while image i computes, image i+1 uploads and the features of image i-1 download. The reference has no host-side
pipeline (single stream, README.md:18); this is an addition for serving throughput.

    pipe = HostPipeline(lambda x: fast.get_intermediate_layers(x, n=[4, 11, 17, 23], return_class_token=True))
    for img in pinned_images:
        ticket = pipe.submit(img)          # returns at once
        ...
        feats = pipe.result(ticket)        # pinned host tensors, valid until `depth` more submissions
"""
import torch


def _map(o, fn):
    if torch.is_tensor(o):
        return fn(o)
    if isinstance(o, (list, tuple)):
        return type(o)(_map(v, fn) for v in o)
    if isinstance(o, dict):
        return {k: _map(v, fn) for k, v in o.items()}
    return o


def _flat(o, out):
    if torch.is_tensor(o):
        out.append(o)
    elif isinstance(o, (list, tuple)):
        for v in o:
            _flat(v, out)
    elif isinstance(o, dict):
        for v in o.values():
            _flat(v, out)
    return out


class HostPipeline:
    def __init__(self, fn, device=None, depth=2):
        if depth < 2:
            raise ValueError("depth must be at least 2 (one buffer computing, one in flight)")
        self.fn, self.depth = fn, depth
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.up, self.down = torch.cuda.Stream(self.device), torch.cuda.Stream(self.device)
        self._x_dev = [None] * depth
        self._host_out = [None] * depth
        self._computed = [None] * depth     # event: compute of the submission using slot s has finished
        self._downloaded = [None] * depth   # event: its features are in host memory
        self._count = 0
        self.h2d_bytes = self.d2h_bytes = 0

    def submit(self, x_host):
        """Enqueue upload -> forward -> download for one host batch (pinned memory makes the copies asynchronous)."""
        s = self._count % self.depth
        main = torch.cuda.current_stream(self.device)
        if self._x_dev[s] is None or self._x_dev[s].shape != x_host.shape or self._x_dev[s].dtype != x_host.dtype:
            self._x_dev[s] = torch.empty(x_host.shape, dtype=x_host.dtype, device=self.device)
        if self._computed[s] is not None:
            self.up.wait_event(self._computed[s])        # the forward that read this input buffer is done
        with torch.cuda.stream(self.up):
            self._x_dev[s].copy_(x_host, non_blocking=True)
            uploaded = torch.cuda.Event()
            uploaded.record(self.up)
        main.wait_event(uploaded)
        out = self.fn(self._x_dev[s])
        computed = torch.cuda.Event()
        computed.record(main)
        self._computed[s] = computed
        if self._host_out[s] is None:
            self._host_out[s] = _map(out, lambda t: torch.empty(t.shape, dtype=t.dtype).pin_memory())
        self.down.wait_event(computed)
        with torch.cuda.stream(self.down):
            for d, h in zip(_flat(out, []), _flat(self._host_out[s], [])):
                d.record_stream(self.down)                # keep the allocator from reusing it before the copy ran
                h.copy_(d, non_blocking=True)
            downloaded = torch.cuda.Event()
            downloaded.record(self.down)
        self._downloaded[s] = downloaded
        self.h2d_bytes = x_host.numel() * x_host.element_size()
        self.d2h_bytes = sum(t.numel() * t.element_size() for t in _flat(out, []))
        self._count += 1
        return self._count - 1

    def result(self, ticket):
        """Block until the features of submission `ticket` are in host memory and return them (pinned buffers that are
        overwritten `depth` submissions later)."""
        if not (self._count - self.depth <= ticket < self._count):
            raise ValueError("ticket is no longer (or not yet) held by the pipeline")
        s = ticket % self.depth
        self._downloaded[s].synchronize()
        return self._host_out[s]

    def drain(self):
        """Make the current stream wait for every outstanding download (so an event recorded on it afterwards covers
        the whole pipeline) and return the last ticket."""
        main = torch.cuda.current_stream(self.device)
        for e in self._downloaded:
            if e is not None:
                main.wait_event(e)
        return self._count - 1
