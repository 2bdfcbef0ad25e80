"""Train-step runner over the C-ABI kernels: the two model families of the
reference's examples, executed the way mograd's scheduler would execute the
simplified forward graph and the gradient sub-graph its rules build.

  * MLP              -- examples/mnist (Linear/ReLU/LayerNorm/Linear + CE)
  * TinyTransformer  -- examples/tinyshakespear/model.mojo:10-130 (Embedding,
    pre-LayerNorm blocks with bias-free Q/K/V/O, ReLU FFN with a bias on W1
    only, untied bias-free lm_head, no positional embedding, no final norm)

All parameters live in one flat buffer (and their gradients in another laid
out the same way), so the optimiser is a single AdamW launch and the
data-parallel exchange is a handful of large NCCL all-reduces over contiguous
slices that are issued while the rest of the backward pass is still running.
PyTorch supplies device memory, streams and the NCCL process group only.
"""
from __future__ import annotations

import ctypes
import os
import math
from dataclasses import dataclass

import torch

from . import _lib
from . import dispatch as K


def _pad8(n: int) -> int:
    return (n + 7) // 8 * 8


class ParamStore:
    """Flat parameter / gradient / optimiser-state buffers with named views."""

    def __init__(self, dtype, device):
        self.dtype = dtype
        self.device = device
        self.specs = []  # (name, shape, offset)
        self.size = 0
        self.aliases = []
        self.alias_parents = []

    def declare(self, name, shape):
        n = 1
        for s in shape:
            n *= s
        off = self.size
        self.specs.append((name, tuple(shape), off))
        self.size = off + (n + 127) // 128 * 128  # keep every tensor 256-byte aligned
        return name

    def allocate(self):
        self.w = torch.zeros(self.size, dtype=self.dtype, device=self.device)
        self.g = torch.zeros(self.size, dtype=self.dtype, device=self.device)
        self.m = torch.zeros(self.size, dtype=torch.float32, device=self.device)
        self.v = torch.zeros(self.size, dtype=torch.float32, device=self.device)
        self.master = torch.zeros(self.size, dtype=torch.float32, device=self.device)
        self.P, self.G, self.range = {}, {}, {}
        for name, shape, off in self.specs:
            n = 1
            for s in shape:
                n *= s
            self.P[name] = self.w[off:off + n].view(shape)
            self.G[name] = self.g[off:off + n].view(shape)
            self.range[name] = (off, off + n)

    def alias(self, name, parent, row_lo, row_hi):
        """Expose rows [row_lo, row_hi) of a declared matrix under a second name (e.g. Wq inside Wqkv)."""
        off, _ = self.range[parent]
        cols = self.P[parent].shape[1]
        self.P[name] = self.P[parent][row_lo:row_hi]
        self.G[name] = self.G[parent][row_lo:row_hi]
        self.range[name] = (off + row_lo * cols, off + row_hi * cols)
        self.aliases.append((name, (row_hi - row_lo, cols)))

    def reference_names(self):
        """(name, shape) of every parameter under the reference model's own names."""
        hidden = {p for p, _ in self.alias_parents}
        out = [(n, shp) for n, shp, _ in self.specs if n not in hidden]
        return out + list(self.aliases)

    def load(self, values: dict):
        """values: name -> float32 CPU tensor; fills master and the working copy."""
        for name, t in values.items():
            off, end = self.range[name]
            self.master[off:end].copy_(t.reshape(-1).to(self.device, torch.float32))
        self.w.copy_(self.master.to(self.dtype))
        self.master.copy_(self.w.float())  # the master starts as the rounded working copy


@dataclass
class AdamWConfig:
    lr: float = 3e-4
    beta1: float = 0.9
    beta2: float = 0.999
    eps: float = 1e-8
    weight_decay: float = 0.1


class _SegmentedStep:
    """Replay of a data-parallel step: its graphs and, between them, the all-reduces of the buckets they complete,
    then AdamW bucket by bucket as each all-reduce finishes (the same order as the kernel-by-kernel step)."""

    def __init__(self, model, segments):
        self.model, self.segments = model, segments

    def replay(self):
        m = self.model
        m._advanced = False
        for kind, what in self.segments:
            if kind == "graph":
                what.replay()
            else:
                for i in what:
                    m._exchange_bucket(i)
        main = torch.cuda.current_stream(m.device)
        for lo, hi, done in m._bucket_done:
            main.wait_event(done)
            m.optimizer_step(lo, hi)
        m._bucket_done.clear()


class _Model:
    """Shared plumbing: flat params, bucketed gradient exchange, optimiser, host-facing step()."""

    def __init__(self, dtype, device, opt: AdamWConfig | None, world_size=1, process_group=None,
                 bucket_bytes=64 << 20):
        self.dtype = dtype
        self.device = torch.device(device)
        self.opt = opt or AdamWConfig()
        self.world_size = world_size
        self.pg = process_group
        self.bucket_bytes = bucket_bytes
        self.store = ParamStore(dtype, self.device)
        self.step_count = 0
        self.comm_stream = None
        self.exchanged = []  # (lo, hi) slices all-reduced so far, in issue order (cleared by the caller)
        self.exchange_enabled = True
        self.time_exposed = False   # record how long the main stream waits for each bucket's all-reduce
        self.exposed_events = []    # per step: [(lo, hi, before, after)] CUDA events around each wait
        self._staged = None         # input slot whose host->device copy has been issued ahead of its step
        self._inflight = None       # (slot, host inputs) of a step that step(launch_next=True) has already queued
        self._slot = 0
        # step() replays a captured CUDA graph of the whole step (one per input slot) after two eager steps: the
        # host then issues one launch per step instead of several hundred, which matters whenever step() must hand
        # the loss back before the next step can be queued.  A data-parallel step is captured as a sequence of
        # graphs cut at the points where a gradient bucket is complete; the all-reduces themselves stay ordinary
        # NCCL calls on the communication stream between the replays (captured together with the step they made the
        # two-GPU test take minutes instead of seconds).  MOGRAD_B200_GRAPH=0 switches the replay off.
        self.use_graph = self.device.type == "cuda" and os.environ.get("MOGRAD_B200_GRAPH", "1") != "0"
        self._cap = None            # state of a segmented capture in progress (data-parallel runs)
        self._graphs = [None, None]
        self._graph_loss = [None, None]
        self.graph_launches = [0, 0]  # kernels of this library recorded in each slot's graph (= launched per replay)
        self._eager_steps = 0
        self._advanced = False      # this step's optimiser launches have already advanced the device step counter
        # dW products on a second stream inside captured steps (see _linear_bwd); MOGRAD_B200_DW_STREAM=0 switches
        # it off
        self.dw_overlap = self.device.type == "cuda" and os.environ.get("MOGRAD_B200_DW_STREAM", "1") != "0"
        self.dw_stream = torch.cuda.Stream(device=self.device) if self.dw_overlap else None
        self._dw_done = {}          # name of the dY buffer -> event: the dW product that reads it has finished
        # 1-based step number on the device: a replayed launch cannot carry a new scalar
        self.d_step = torch.zeros(1, dtype=torch.int32, device=self.device) if self.device.type == "cuda" else None

    # ---- host-side input staging ---------------------------------------------------------
    def _setup_io(self, in_shape, in_dtype, tgt_shape):
        """Two device slots for the batch (the copy of step k+1 may run while step k computes), each with a pinned
        word for the loss and pinned words for the device status of the step that reads it."""
        dev = self.device
        self._in = [torch.empty(in_shape, dtype=in_dtype, device=dev) for _ in range(2)]
        self._tgt = [torch.empty(tgt_shape, dtype=torch.int64, device=dev) for _ in range(2)]
        self.d_inputs, self.d_targets = self._in[0], self._tgt[0]
        on_gpu = dev.type == "cuda"
        # per input slot: pinned result words and an event recorded behind each step that reads the slot
        self._h_loss = [torch.empty((), dtype=torch.float32).pin_memory() for _ in range(2)] if on_gpu else None
        self._h_status = [torch.zeros(4, dtype=torch.int32).pin_memory() for _ in range(2)] if on_gpu else None
        self._done = [torch.cuda.Event() for _ in range(2)] if on_gpu else None
        self.copy_stream = torch.cuda.Stream(device=dev) if on_gpu else None
        self._copied = [None, None]  # event per slot: its host->device copy has finished

    def use_slot(self, k: int):
        """Make input slot k (0 or 1) the batch the next step_device() reads."""
        self._slot = k
        self.d_inputs, self.d_targets = self._in[k], self._tgt[k]

    def _prefetch(self, host_inputs, host_targets):
        """Issue the host->device copy of the next step's batch on the copy stream, into the slot the current step
        is not using (that slot was last read by the step before this one, which step() has synchronised with)."""
        k = self._slot ^ 1
        cs = self.copy_stream
        with torch.cuda.stream(cs):
            self._in[k].copy_(host_inputs, non_blocking=True)
            self._tgt[k].copy_(host_targets, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(cs)
        self._copied[k] = ev
        self._staged = (k, host_inputs)

    # ---- data-parallel gradient exchange -------------------------------------------------
    def _setup_buckets(self):
        if self.world_size > 1 and self.device.type == "cuda":
            self.comm_stream = torch.cuda.Stream(device=self.device)
        esz = self.store.g.element_size()
        per = max(1, self.bucket_bytes // esz)
        # buckets are contiguous slices; gradients are produced from the end of the buffer backwards
        self.buckets = []
        hi = self.store.size
        while hi > 0:
            lo = max(0, (hi - per) // 128 * 128)  # 128-element boundaries keep every slice 16-byte aligned
            self.buckets.append((lo, hi))
            hi = lo
        self._next_bucket = 0
        self._bucket_done = []  # (lo, hi, event recorded on the communication stream after the bucket's all-reduce)

    def _grads_ready_down_to(self, offset: int):
        """Everything in the flat gradient buffer at or above `offset` is final: exchange the buckets it covers."""
        if self.world_size == 1 or not self.exchange_enabled:
            return
        import torch.distributed as dist

        ready = []
        while self._next_bucket < len(self.buckets) and self.buckets[self._next_bucket][0] >= offset:
            ready.append(self._next_bucket)
            self._next_bucket += 1
        if not ready:
            return
        if self._cap is not None:
            # a step is being captured: close the graph that produced these buckets, note the exchange to be issued
            # at this point of every replay, open the next graph
            self._end_segment()
            self._cap["segments"].append(("exchange", ready))
            self._begin_segment()
            return
        for i in ready:
            self._exchange_bucket(i)

    def _exchange_bucket(self, i):
        import torch.distributed as dist

        lo, hi = self.buckets[i]
        if self.comm_stream is None:  # host tensors (gloo): no streams to order
            dist.all_reduce(self.store.g[lo:hi], op=dist.ReduceOp.SUM, group=self.pg)
        else:
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream(self.device))
            self.comm_stream.wait_event(ev)
            with torch.cuda.stream(self.comm_stream):
                dist.all_reduce(self.store.g[lo:hi], op=dist.ReduceOp.SUM, group=self.pg)
                done = torch.cuda.Event()
                done.record(self.comm_stream)
            self._bucket_done.append((lo, hi, done))
        self.exchanged.append((lo, hi))

    def _finish_exchange(self):
        if self.world_size == 1:
            return
        self._grads_ready_down_to(0)
        if self.comm_stream is not None:
            torch.cuda.current_stream(self.device).wait_stream(self.comm_stream)
        self._next_bucket = 0

    def optimizer_step(self, lo=0, hi=None):
        """AdamW on the flat range [lo, hi) (everything by default); the caller advances step_count."""
        o = self.opt
        s = self.store
        hi = s.size if hi is None else hi
        if self.d_step is not None:
            K.adamw_step_dev(s.w[lo:hi], s.g[lo:hi], s.m[lo:hi], s.v[lo:hi], s.master[lo:hi], o.lr, o.beta1, o.beta2,
                             o.eps, o.weight_decay, self.d_step, not self._advanced, grad_scale=1.0 / self.world_size)
            self._advanced = True
        else:
            K.adamw_step(s.w[lo:hi], s.g[lo:hi], s.m[lo:hi], s.v[lo:hi], s.master[lo:hi], o.lr, o.beta1, o.beta2,
                         o.eps, o.weight_decay, self.step_count, grad_scale=1.0 / self.world_size)

    # ---- backward of a linear layer, dW optionally on its own stream -----------------------
    def _linear_bwd(self, tag, dy, x, w, dx_out, dw_out, db_out=None, **kw):
        """dX on the current stream; dW (and db) either behind it or, with dw_overlap, on a second stream that only
        waits for dY: nothing downstream needs dW before the optimiser, so its CTAs can fill the SMs that the tail
        wave of the dX chain leaves idle.  `tag` names the dY buffer; _dy_free(tag) must precede whatever overwrites
        that buffer."""
        # only while a step is being captured into a graph: launched kernel by kernel, the extra event records and
        # waits cost the host more than the overlap gives the device on small models
        if not (self.dw_overlap and torch.cuda.is_current_stream_capturing()):
            K.matmul_bias_bt_bwd(dy, x, w, dx_out=dx_out, dw_out=dw_out, db_out=db_out, need_db=db_out is not None, **kw)
            return
        main = torch.cuda.current_stream(self.device)
        ready = torch.cuda.Event()
        ready.record(main)
        K.matmul_bias_bt_bwd(dy, x, w, dx_out=dx_out, need_dw=False, need_db=False, **kw)
        side = self.dw_stream
        side.wait_event(ready)
        with torch.cuda.stream(side):
            K.matmul_bias_bt_bwd(dy, x, w, need_dx=False, dw_out=dw_out, db_out=db_out, need_db=db_out is not None)
            done = torch.cuda.Event()
            done.record(side)
        self._dw_done[tag] = done

    def _dy_free(self, tag):
        ev = self._dw_done.pop(tag, None)
        if ev is not None:
            torch.cuda.current_stream(self.device).wait_event(ev)

    def _dw_join(self):
        for tag in list(self._dw_done):
            self._dy_free(tag)

    # ---- host-facing call: host buffers in, loss out -------------------------------------
    def step(self, host_inputs, host_targets, prefetch=None, launch_next=False) -> float:
        """One train step from pinned host tensors; returns the loss as a Python float (device->host read).

        prefetch=(next_inputs, next_targets): the next step's batch; its host->device copy is issued on a second
        stream right after this step's kernels are queued, so it runs under them, and the next step(next_inputs,
        ...) finds its batch on the device.

        launch_next=True (with prefetch) commits to that next step: it is queued behind this one before this call
        waits for its own loss, so the device never idles between steps while the host reads a result and queues
        the next step (one graph launch on a single GPU, several hundred kernel launches otherwise); the call
        still returns this step's loss (each input slot has pinned result words of its own).  The caller must then
        make its next call step(next_inputs, next_targets, ...).

        Raises KernelError when a kernel's bounded wait gave up during the step (the status word rides back with
        the loss)."""
        main = torch.cuda.current_stream(self.device)
        if self._inflight is not None:
            k, expected = self._inflight
            self._inflight = None
            if expected is not host_inputs:
                raise ValueError("Model.step: the previous call committed to a different next batch (launch_next)")
            self.use_slot(k)
        else:
            if self._staged is not None and self._staged[1] is host_inputs:
                k, self._staged = self._staged[0], None
                self.use_slot(k)
                main.wait_event(self._copied[k])
            else:
                self._staged = None
                self.d_inputs.copy_(host_inputs, non_blocking=True)
                self.d_targets.copy_(host_targets, non_blocking=True)
            k = self._slot
            self._launch(k)
        if prefetch is not None:
            self._prefetch(*prefetch)
            if launch_next:
                # the next step, queued now: its batch copy is ordered before it by the slot's event
                kn = k ^ 1
                main.wait_event(self._copied[kn])
                self._launch(kn)
                self.use_slot(k)
                self._inflight, self._staged = (kn, prefetch[0]), None
        self._done[k].synchronize()
        if int(self._h_status[k][0]) != 0:
            _lib.check_device_status("Model.step")
        return float(self._h_loss[k].item())

    def _launch(self, k):
        """Queues one step on the batch in input slot k (graph replay when the slot's graph exists, kernel by kernel
        otherwise), the copies of its loss and of the device status to the slot's pinned words, and the slot's
        event behind them."""
        main = torch.cuda.current_stream(self.device)
        self.use_slot(k)
        if self.use_graph and self._graphs[k] is None and self._eager_steps >= 2:
            self._capture(k)
        if self.use_graph and self._graphs[k] is not None:
            self._graphs[k].replay()
            self.step_count += 1
        else:
            loss = self.step_device()
            self._eager_steps += 1
            self._h_loss[k].copy_(loss, non_blocking=True)
            _lib.call("mograd_b200_device_status_async", ctypes.c_void_p(self._h_status[k].data_ptr()),
                      ctypes.c_void_p(main.cuda_stream))
        self._done[k].record(main)

    def _begin_segment(self):
        g = torch.cuda.CUDAGraph()
        # thread-local mode: NCCL's watchdog thread makes CUDA calls of its own while this thread captures
        g.capture_begin(pool=self._cap["pool"], capture_error_mode="thread_local")
        self._cap["graph"] = g

    def _end_segment(self):
        self._dw_join()  # streams forked inside a graph are joined inside it
        self._cap["graph"].capture_end()
        self._cap["segments"].append(("graph", self._cap["graph"]))

    def _capture_segments(self, k):
        """Data-parallel form of _capture: the forward and backward pass of a step reading input slot k as a sequence
        of graphs cut wherever a gradient bucket is complete, with the bucket's all-reduce noted between them; the
        replay object issues graphs and all-reduces in that order and then the per-bucket optimiser launches."""
        main = torch.cuda.current_stream(self.device)
        side = torch.cuda.Stream(device=self.device)
        torch.cuda.synchronize(self.device)
        side.wait_stream(main)
        count = self.step_count
        n0 = _lib.load().mograd_b200_launch_count()
        self._cap = dict(pool=torch.cuda.graph_pool_handle(), segments=[], graph=None)
        self._next_bucket = 0
        try:
            with torch.cuda.stream(side):
                self._begin_segment()
                loss = self.forward_backward()
                self._grads_ready_down_to(0)
                self._h_loss[k].copy_(loss, non_blocking=True)
                _lib.call("mograd_b200_device_status_async", ctypes.c_void_p(self._h_status[k].data_ptr()),
                          ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream))
                self._end_segment()
            segments = self._cap["segments"]
        finally:
            self._cap = None
            self._next_bucket = 0
        self.step_count = count
        self.graph_launches[k] = int(_lib.load().mograd_b200_launch_count() - n0)
        main.wait_stream(side)
        self._graphs[k], self._graph_loss[k] = _SegmentedStep(self, segments), loss

    def _capture(self, k):
        """Records one whole step reading input slot k (kernels, the loss and status copies to pinned host words)
        into a CUDA graph.  Nothing runs during the capture; the caller replays it."""
        if self.world_size > 1:
            return self._capture_segments(k)
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        g = torch.cuda.CUDAGraph()
        count = self.step_count
        n0 = _lib.load().mograd_b200_launch_count()
        with torch.cuda.graph(g, stream=side):
            loss = self.step_device()
            self._h_loss[k].copy_(loss, non_blocking=True)
            _lib.call("mograd_b200_device_status_async", ctypes.c_void_p(self._h_status[k].data_ptr()),
                      ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream))
        self.step_count = count  # the capture executed nothing
        self.graph_launches[k] = int(_lib.load().mograd_b200_launch_count() - n0)
        torch.cuda.current_stream(self.device).wait_stream(side)
        self._graphs[k], self._graph_loss[k] = g, loss

    def step_resident(self, k: int):
        """One train step on the batch already resident in input slot k, no host input or output: replays the
        slot's captured graph (captured on first use after two eager steps) or, without graphs, launches the step
        kernel by kernel.  Returns the loss as a device tensor."""
        self.use_slot(k)
        if self.use_graph and self._graphs[k] is None and self._eager_steps >= 2:
            self._capture(k)
        if self.use_graph and self._graphs[k] is not None:
            self._graphs[k].replay()
            self.step_count += 1
            return self._graph_loss[k]
        self._eager_steps += 1
        return self.step_device()

    def step_device(self):
        self._advanced = False
        loss = self.forward_backward()
        self.step_count += 1
        if self.world_size > 1 and self.comm_stream is not None:
            # The optimiser follows the exchange bucket by bucket: buckets reduced during the backward pass are
            # updated while the last ones (the embedding gradient, final only when the backward pass ends) are
            # still on the wire.
            self._grads_ready_down_to(0)
            main = torch.cuda.current_stream(self.device)
            marks = []
            for lo, hi, done in self._bucket_done:
                if self.time_exposed:
                    before = torch.cuda.Event(enable_timing=True)
                    before.record(main)
                main.wait_event(done)
                if self.time_exposed:
                    after = torch.cuda.Event(enable_timing=True)
                    after.record(main)
                    marks.append((lo, hi, before, after))
                self.optimizer_step(lo, hi)
            if self.time_exposed:
                self.exposed_events.append(marks)
            self._bucket_done.clear()
            self._next_bucket = 0
        else:
            self._finish_exchange()
            self.optimizer_step()
        return loss


    # ---- data-parallel self-check ---------------------------------------------------------
    def check_data_parallel(self):
        """Compares the bucketed, overlapped gradient exchange with a plain one on the current batch.

        Runs forward+backward twice without touching the parameters: once with the exchange switched off (the
        local gradients, summed over ranks in fp32 by a single all-reduce on the main stream) and once through
        the product path (bf16 buckets on the communication stream behind events).  Returns
        max |product - plain| / max |plain| over the whole flat gradient buffer, the same on every rank."""
        import torch.distributed as dist

        if self.world_size == 1:
            return 0.0
        self.exchange_enabled = False
        self.forward_backward()
        self.exchange_enabled = True
        plain = self.store.g.float()
        dist.all_reduce(plain, op=dist.ReduceOp.SUM, group=self.pg)
        self.forward_backward()
        self._finish_exchange()
        self._bucket_done.clear()
        got = self.store.g.float()
        err = (got - plain).abs().max() / plain.abs().max().clamp_min(1e-30)
        dist.all_reduce(err, op=dist.ReduceOp.MAX, group=self.pg)
        return float(err.item())

    def replicas_in_sync(self):
        """True when every rank holds bit-identical parameters and optimiser master copies."""
        import torch.distributed as dist

        if self.world_size == 1:
            return True
        w = self.store.w.view(torch.int16).to(torch.int64)
        sums = torch.stack([w.sum(), (w * w).sum(), self.store.master.view(torch.int32).to(torch.int64).sum()])
        lo, hi = sums.clone(), sums.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN, group=self.pg)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX, group=self.pg)
        return bool(torch.equal(lo, hi))


class MLP(_Model):
    """Linear(d0->d1)+ReLU -> LayerNorm(d1) -> [Linear+ReLU]* -> Linear(->classes), cross-entropy loss."""

    def __init__(self, dims, batch, dtype=torch.bfloat16, device="cuda", opt=None, seed=0, **kw):
        super().__init__(dtype, device, opt, **kw)
        self.dims = list(dims)
        self.batch = batch
        self.nl = len(dims) - 1
        st = self.store
        for i in range(self.nl):
            st.declare(f"W{i}", (dims[i + 1], dims[i]))
            st.declare(f"b{i}", (dims[i + 1],))
            if i == 0:
                st.declare("ln_g", (dims[1],))
                st.declare("ln_b", (dims[1],))
        st.allocate()
        g = torch.Generator().manual_seed(seed)
        vals = {}
        for i in range(self.nl):
            bound = 1.0 / math.sqrt(dims[i])
            vals[f"W{i}"] = (torch.rand((dims[i + 1], dims[i]), generator=g) * 2 - 1) * bound
            vals[f"b{i}"] = (torch.rand((dims[i + 1],), generator=g) * 2 - 1) * bound
        vals["ln_g"] = torch.ones(dims[1])
        vals["ln_b"] = torch.zeros(dims[1])
        st.load(vals)
        self._setup_buckets()
        dev, B = self.device, batch
        self._setup_io((B, dims[0]), dtype, (B,))
        self.act = [torch.empty((B, dims[i + 1]), dtype=dtype, device=dev) for i in range(self.nl - 1)]
        self.ln_out = torch.empty((B, dims[1]), dtype=dtype, device=dev)
        self.C = dims[-1]
        self.logits_buf = torch.empty((B, _pad8(self.C)), dtype=dtype, device=dev)
        self.logits = self.logits_buf[:, :self.C]
        self.dact = [torch.empty((B, dims[i + 1]), dtype=dtype, device=dev) for i in range(self.nl - 1)]
        self.dln = torch.empty((B, dims[1]), dtype=dtype, device=dev)

    def forward_backward(self):
        P, G = self.store.P, self.store.G
        x = self.d_inputs
        # forward
        K.matmul_bias_strided(x, P["W0"], P["b0"], act=1, out=self.act[0])
        K.layer_norm_fwd_dispatch(self.act[0], P["ln_g"], P["ln_b"], out=self.ln_out)
        h = self.ln_out
        for i in range(1, self.nl - 1):
            K.matmul_bias_strided(h, P[f"W{i}"], P[f"b{i}"], act=1, out=self.act[i])
            h = self.act[i]
        K.matmul_bias_strided(h, P[f"W{self.nl - 1}"], P[f"b{self.nl - 1}"], out=self.logits)
        loss, dl = K.softmax_xent_fwd_bwd(self.logits, self.d_targets, inplace=True)
        # backward
        dy = dl
        for i in range(self.nl - 1, 0, -1):
            inp = self.act[i - 1] if i > 1 else self.ln_out
            dst = self.dact[i - 1] if i > 1 else self.dln
            self._linear_bwd(f"dy{i}", dy, inp, P[f"W{i}"], dst, G[f"W{i}"], db_out=G[f"b{i}"],
                             relu_y=self.act[i - 1] if i > 1 else None)
            self._grads_ready_down_to(self.store.range[f"W{i}"][0])
            dy = dst
        K.layer_norm_bwd_dispatch(self.dln, self.act[0], P["ln_g"], dx_out=self.dln, dgamma_out=G["ln_g"],
                                  dbeta_out=G["ln_b"])
        K.relu_grad(self.act[0], self.dln)
        K.matmul_bias_bt_bwd(self.dln, x, P["W0"], need_dx=False, dw_out=G["W0"], db_out=G["b0"])
        self._dw_join()
        return loss


class TinyTransformer(_Model):
    """Decoder-only transformer of examples/tinyshakespear/model.mojo, one train step at a time.

    W_Q, W_K and W_V of a block are stored as the three row blocks of one (3d, d) matrix, so their three
    projections (and the three dX / dW products of the backward pass) run as single GEMMs; attention reads Q, K, V
    as column blocks of that GEMM's output and writes its output token-major, so no transpose copy is needed.
    """

    def __init__(self, vocab, d_model, d_ff, n_layers, n_heads, batch, seq, dtype=torch.bfloat16, device="cuda",
                 opt=None, seed=0, init_std=0.02, **kw):
        super().__init__(dtype, device, opt, **kw)
        self.V, self.d, self.dff, self.L, self.H = vocab, d_model, d_ff, n_layers, n_heads
        self.B, self.S = batch, seq
        self.Dh = d_model // n_heads
        self.T = batch * seq
        st = self.store
        st.declare("embed", (vocab, d_model))
        for l in range(n_layers):
            st.declare(f"Wqkv{l}", (3 * d_model, d_model))
            st.alias_parents.append((f"Wqkv{l}", l))
            st.declare(f"Wo{l}", (d_model, d_model))
            st.declare(f"W1_{l}", (d_ff, d_model))
            st.declare(f"b1_{l}", (d_ff,))
            st.declare(f"W2_{l}", (d_model, d_ff))
            for nm in ("g1", "be1", "g2", "be2"):
                st.declare(f"{nm}_{l}", (d_model,))
        st.declare("lm_head", (vocab, d_model))
        st.allocate()
        for l in range(n_layers):
            for r, nm in enumerate(("Wq", "Wk", "Wv")):
                st.alias(f"{nm}{l}", f"Wqkv{l}", r * d_model, (r + 1) * d_model)
        g = torch.Generator().manual_seed(seed)
        vals = {}
        for name, shape, _ in st.specs:
            if name.startswith(("g1_", "g2_")):
                vals[name] = torch.ones(shape)
            elif name.startswith(("be1_", "be2_", "b1_")):
                vals[name] = torch.zeros(shape)
            else:
                vals[name] = torch.randn(shape, generator=g) * init_std
        st.load(vals)
        self._setup_buckets()
        dev, T, d = self.device, self.T, d_model
        new = lambda *shape: torch.empty(shape, dtype=dtype, device=dev)
        self._setup_io((batch, seq), torch.int64, (batch, seq))
        self.x = [new(T, d) for _ in range(n_layers + 1)]  # block inputs, x[L] = final hidden state
        self.saved = []
        for _ in range(n_layers):
            self.saved.append(dict(ln1=new(T, d), qkv=new(T, 3 * d), ctx=new(T, d),
                                   lse=torch.empty((batch, n_heads, seq), dtype=torch.float32, device=dev),
                                   h=new(T, d), ln2=new(T, d), f1=new(T, d_ff)))
        # ReLU mask of the feed-forward activation as one bit per element (16-bit tensor-core path only): the backward
        # GEMM fetches T*d_ff/8 bytes instead of re-reading the activation
        self.relu_bits = dtype in (torch.bfloat16, torch.float16) and dev.type == "cuda" and d % 8 == 0 and d_ff % 8 == 0
        if self.relu_bits:
            for sv in self.saved:
                sv["f1_bits"] = torch.empty((T, (d_ff + 31) // 32), dtype=torch.int32, device=dev)
        self.Vp = _pad8(vocab)
        self.logits_buf = new(T, self.Vp)
        self.logits = self.logits_buf[:, :vocab]
        # backward scratch, reused by every block
        self.t_dx, self.t_b = new(T, d), new(T, d)
        self.t_ff = new(T, d_ff)
        self.t_dqkv = new(T, 3 * d)

    def _heads(self, qkv):
        """(q, k, v) views (B, S, H, Dh) of a (T, 3d) fused projection buffer."""
        v5 = qkv.view(self.B, self.S, 3, self.H, self.Dh)
        return v5[:, :, 0], v5[:, :, 1], v5[:, :, 2]

    def forward_backward(self):
        P, G, st = self.store.P, self.store.G, self.store
        B, S, H, Dh, L = self.B, self.S, self.H, self.Dh, self.L
        tok = self.d_inputs.view(-1)
        K.gather_rows(P["embed"], tok, out=self.x[0])
        for l in range(L):
            sv, x = self.saved[l], self.x[l]
            K.layer_norm_fwd_dispatch(x, P[f"g1_{l}"], P[f"be1_{l}"], out=sv["ln1"])
            K.matmul_bias_strided(sv["ln1"], P[f"Wqkv{l}"], out=sv["qkv"])
            q4, k4, v4 = self._heads(sv["qkv"])
            K.flash_attn_fwd_dispatch(q4, k4, v4, None, None, True, False, out=sv["ctx"].view(B, S, H, Dh),
                                      lse_out=sv["lse"], o_bshd=True)
            K.matmul_bias_strided(sv["ctx"], P[f"Wo{l}"], out=sv["h"], residual=x)
            K.layer_norm_fwd_dispatch(sv["h"], P[f"g2_{l}"], P[f"be2_{l}"], out=sv["ln2"])
            K.matmul_bias_strided(sv["ln2"], P[f"W1_{l}"], P[f"b1_{l}"], act=1, out=sv["f1"],
                                  relu_bits=sv.get("f1_bits"))
            K.matmul_bias_strided(sv["f1"], P[f"W2_{l}"], out=self.x[l + 1], residual=sv["h"])
        K.matmul_bias_strided(self.x[L], P["lm_head"], out=self.logits)
        loss, dl = K.softmax_xent_fwd_bwd(self.logits, self.d_targets.view(-1), inplace=True)

        # ---- backward
        dx = self.t_dx  # gradient w.r.t. the current block's output
        self._linear_bwd("dl", dl, self.x[L], P["lm_head"], dx, G["lm_head"])
        self._grads_ready_down_to(st.range["lm_head"][0])
        for l in range(L - 1, -1, -1):
            sv, x = self.saved[l], self.x[l]
            # FFN: out = h + W2 relu(W1 ln2 + b1)
            self._dy_free("t_ff")  # the previous block's W1 dW has read t_ff
            self._linear_bwd("dx", dx, sv["f1"], P[f"W2_{l}"], self.t_ff, G[f"W2_{l}"],
                             relu_y=None if self.relu_bits else sv["f1"], relu_bits=sv.get("f1_bits"))
            self._linear_bwd("t_ff", self.t_ff, sv["ln2"], P[f"W1_{l}"], self.t_b, G[f"W1_{l}"], db_out=G[f"b1_{l}"])
            self._dy_free("dx")
            K.layer_norm_bwd_dispatch(self.t_b, sv["h"], P[f"g2_{l}"], dx_out=dx, dgamma_out=G[f"g2_{l}"],
                                      dbeta_out=G[f"be2_{l}"], dx_residual=dx)  # dx is now dL/dh
            # attention: h = x + Wo ctx
            self._linear_bwd("dx", dx, sv["ctx"], P[f"Wo{l}"], self.t_b, G[f"Wo{l}"])
            q4, k4, v4 = self._heads(sv["qkv"])
            self._dy_free("t_dqkv")  # the previous block's Wqkv dW has read t_dqkv
            K.flash_attn_bwd_dispatch(self.t_b.view(B, S, H, Dh), sv["ctx"].view(B, S, H, Dh), q4, k4, v4, None,
                                      sv["lse"], None, True, False, out=self._heads(self.t_dqkv), o_bshd=True)
            self._linear_bwd("t_dqkv", self.t_dqkv, sv["ln1"], P[f"Wqkv{l}"], self.t_b, G[f"Wqkv{l}"])
            self._dy_free("dx")
            K.layer_norm_bwd_dispatch(self.t_b, x, P[f"g1_{l}"], dx_out=dx, dgamma_out=G[f"g1_{l}"],
                                      dbeta_out=G[f"be1_{l}"], dx_residual=dx)  # dx is now dL/dx
            self._grads_ready_down_to(st.range[f"Wqkv{l}"][0])
        K.scatter_add_rows(dx, tok, self.V, out=G["embed"])
        self._dw_join()
        return loss
