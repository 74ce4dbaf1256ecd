"""Data-parallel gradient exchange for the linear-layer path.

The GEMM rows (B*T) are independent across sequences, so N GPUs each run the same GEMM set on
their own batch and only the weight/bias gradients cross the links: one averaged all-reduce
per bucket (NCCL over NVLink on GPUs, gloo in the CPU tests). Buckets are handed over in the
order the backward pass finishes them, each on a side stream behind an event, so that the
exchange of bucket i runs under the backward_weight GEMMs of bucket i+1.

The reference is single-GPU (no collective anywhere in vnnm404/gpt2.cu); its flat gradient
buffer g_model.params_memory (include/gpt2/gpt2.h:70) is what these buckets slice.
"""
import torch
import torch.distributed as dist


def compute_stream(handle=None):
    """The torch stream object for a raw cudaStream_t handle (None / 0 = torch's current stream), so that
    events and collectives are ordered against the stream the model's kernels are actually enqueued on."""
    if not handle:
        return torch.cuda.current_stream()
    cur = torch.cuda.current_stream()
    if cur.cuda_stream == handle:
        return cur
    return torch.cuda.ExternalStream(handle)


def plan_buckets(named_sizes, bucket_bytes):
    """Groups (name, numel) pairs, kept in the given order, into buckets of at most
    `bucket_bytes` (fp32); a tensor larger than the limit gets a bucket of its own.
    Returns a list of lists of names."""
    buckets, cur, cur_bytes = [], [], 0
    for name, numel in named_sizes:
        nbytes = 4 * int(numel)
        if cur and cur_bytes + nbytes > bucket_bytes:
            buckets.append(cur)
            cur, cur_bytes = [], 0
        cur.append(name)
        cur_bytes += nbytes
    if cur:
        buckets.append(cur)
    return buckets


class GradientExchange:
    """Averages gradient tensors across the ranks of `group`, overlapped with compute.

    exchange(tensors) is called right after the kernels that produce `tensors` were enqueued on
    the current stream; finish() makes the current stream wait for every exchange issued so far.
    With world_size 1 both are no-ops (nothing to exchange)."""

    def __init__(self, group=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.comm_stream = None
        self.pending = []
        self.calls = 0

    def exchange(self, tensors, stream=None, tag=None):
        """`stream`: raw handle of the stream the producing kernels were enqueued on (default: torch's
        current stream). `tag` is handed back by wait_next()."""
        if self.world == 1:
            return
        tensors = [t for t in tensors if t is not None]
        if not tensors:
            return
        self.calls += 1
        if tensors[0].is_cuda:
            if self.comm_stream is None:
                self.comm_stream = torch.cuda.Stream()
            ready = torch.cuda.Event()
            ready.record(compute_stream(stream))
            with torch.cuda.stream(self.comm_stream):
                self.comm_stream.wait_event(ready)
                for t in tensors:
                    dist.all_reduce(t, op=dist.ReduceOp.AVG, group=self.group)
                done = torch.cuda.Event()
                done.record()
            self.pending.append((done, tag))
        else:
            # gloo has no AVG: sum, then scale
            for t in tensors:
                dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.group)
                t.div_(self.world)
            self.pending.append((None, tag))

    def wait_next(self, stream=None):
        """Makes the compute stream wait for the OLDEST exchange still pending and returns its tag (None when
        nothing is pending): lets the caller consume buckets in the order they were handed over, e.g. run the
        optimizer on bucket i while bucket i+1 is still on the links."""
        if not self.pending:
            return None
        ev, tag = self.pending.pop(0)
        if ev is not None:
            compute_stream(stream).wait_event(ev)
        return tag

    def finish(self, stream=None):
        for ev, _ in self.pending:
            if ev is not None:
                compute_stream(stream).wait_event(ev)
        self.pending = []


def shard_bounds(lo, hi, world):
    """Splits floats [lo, hi) among `world` ranks: rank r owns [lo + r*per, lo + (r+1)*per); the
    remainder [body_end, hi) (fewer than `world` floats) is kept replicated. Returns (per, body_end)."""
    per = (hi - lo) // world
    return per, lo + per * world


class ShardedExchange:
    """Optimizer-state sharding over the flat buffers (ZeRO stage 1 style): gradients are
    reduce-scattered instead of all-reduced, every rank runs AdamW on its own slice of each bucket
    only, and the updated parameter slices are all-gathered. Bytes on the links are the same as an
    all-reduce; the update touches 1/world of the parameters per rank.

    reduce(lo, hi) is called right after the kernels producing grads[lo:hi] were enqueued; it runs on
    a side stream (GPU) like GradientExchange. owned() lists the (first, count) ranges this rank must
    update once finish() has been called; gather() then rebuilds the full parameters everywhere.
    The reference updates the whole buffer on its one GPU (gpt2_update, src/train.cu:450-481)."""

    def __init__(self, grads, params, group=None):
        self.grads, self.params, self.group = grads, params, group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.comm_stream = None
        self.pending = []
        self.ranges = []
        self.calls = 0

    def _mine(self, lo, per):
        return lo + self.rank * per, lo + (self.rank + 1) * per

    def reduce(self, lo, hi, stream=None):
        self.ranges.append((lo, hi))
        if self.world == 1:
            return
        self.calls += 1
        per, body_end = shard_bounds(lo, hi, self.world)
        a, b = self._mine(lo, per)

        def issue():
            if per:
                if self.grads.is_cuda:
                    dist.reduce_scatter_tensor(self.grads[a:b], self.grads[lo:body_end], op=dist.ReduceOp.AVG,
                                               group=self.group)
                else:  # gloo has no AVG
                    dist.reduce_scatter_tensor(self.grads[a:b], self.grads[lo:body_end], op=dist.ReduceOp.SUM,
                                               group=self.group)
                    self.grads[a:b].div_(self.world)
            if body_end < hi:
                if self.grads.is_cuda:
                    dist.all_reduce(self.grads[body_end:hi], op=dist.ReduceOp.AVG, group=self.group)
                else:
                    dist.all_reduce(self.grads[body_end:hi], op=dist.ReduceOp.SUM, group=self.group)
                    self.grads[body_end:hi].div_(self.world)

        if self.grads.is_cuda:
            if self.comm_stream is None:
                self.comm_stream = torch.cuda.Stream()
            ready = torch.cuda.Event()
            ready.record(compute_stream(stream))
            with torch.cuda.stream(self.comm_stream):
                self.comm_stream.wait_event(ready)
                issue()
                done = torch.cuda.Event()
                done.record()
            self.pending.append(done)
        else:
            issue()

    def finish(self, stream=None):
        for ev in self.pending:
            compute_stream(stream).wait_event(ev)
        self.pending = []

    def owned(self):
        """(first, count) ranges whose gradients are final on this rank: its slice of every bucket
        plus the replicated remainders."""
        out = []
        for lo, hi in self.ranges:
            if self.world == 1:
                out.append((lo, hi - lo))
                continue
            per, body_end = shard_bounds(lo, hi, self.world)
            a, b = self._mine(lo, per)
            if per:
                out.append((a, per))
            if body_end < hi:
                out.append((body_end, hi - body_end))
        return out

    def gather(self, stream=None):
        """After the update of owned(): every rank receives the other ranks' parameter slices (issued on
        the compute stream, behind the update kernels)."""
        if self.world > 1:
            ctx = torch.cuda.stream(compute_stream(stream)) if self.params.is_cuda else _NullContext()
            with ctx:
                for lo, hi in self.ranges:
                    per, body_end = shard_bounds(lo, hi, self.world)
                    if not per:
                        continue
                    a, b = self._mine(lo, per)
                    src = self.params[a:b] if self.params.is_cuda else self.params[a:b].clone()
                    dist.all_gather_into_tensor(self.params[lo:body_end], src, group=self.group)
        self.ranges = []


class _NullContext:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


class _DeviceView:
    """Exposes a raw device pointer of `count` fp32 values through __cuda_array_interface__."""

    def __init__(self, ptr, count):
        self.__cuda_array_interface__ = {"shape": (int(count),), "typestr": "<f4", "data": (int(ptr), False),
                                         "version": 3, "strides": None}


def device_tensor(ptr, count, device):
    """A torch tensor aliasing `count` floats at device address `ptr` (no copy, no ownership)."""
    return torch.as_tensor(_DeviceView(ptr, count), device=device)


class DataParallelStep:
    """One data-parallel training step of a gpt2_model (include/gpt2_model.h) per call.

    Every rank runs the forward and backward pass on its own batch; the flat gradient buffer is
    averaged across ranks in buckets, in the order the backward pass completes them — ln_f with the
    last block, then one bucket per block going down, then wte + wpe after the embedding backward —
    each on the side stream while the next block's backward runs on the compute stream (the
    backward_weight GEMMs of block l-1 hide the exchange of block l). AdamW runs replicated, bucket by
    bucket in hand-over order as each all-reduce lands (gpt2_model_update_range), so the update of the
    earlier buckets runs while the last and largest one (wte + wpe) is still on the links. With one rank the
    exchange is a no-op and the update is one call.

    use_graph=True (single rank only): forward + backward are replayed from a CUDA graph
    (gpt2_model_forward_backward_graph), which pays at small shapes where launches dominate.

    shard_optimizer=True swaps the all-reduce for ShardedExchange: reduce-scatter per bucket, AdamW on
    this rank's slices only (gpt2_model_update_range), all-gather of the parameters."""

    def __init__(self, model, device, group=None, shard_optimizer=False, use_graph=False):
        self.model = model
        self.use_graph = use_graph
        self.exchange = GradientExchange(group)
        self.sharded = None
        if shard_optimizer:
            self.sharded = ShardedExchange(device_tensor(model.grads_ptr(), model.num_params, device),
                                           device_tensor(model.params_ptr(), model.num_params, device), group)
        self.L = model.cfg.n_layer
        offs = model.offsets() + [model.num_params]
        self.flat = device_tensor(model.grads_ptr(), model.num_params, device)
        # tensor index: 0 wte, 1 wpe, 2 + 12*l ... block l, then ln_f.w, ln_f.b
        self.block = [(offs[2 + 12 * l], offs[2 + 12 * (l + 1)]) for l in range(self.L)]
        self.embed = (offs[0], offs[2])
        self.lnf = (offs[2 + 12 * self.L], offs[-1])

    def _slice(self, rng):
        return self.flat[rng[0]:rng[1]]

    def __call__(self, tokens, targets, lr, beta1, beta2, eps, weight_decay, t, stream=None):
        m = self.model
        if self.sharded is not None:
            return self._sharded_step(tokens, targets, lr, beta1, beta2, eps, weight_decay, t, stream)
        if self.exchange.world == 1 and self.use_graph:
            # nothing to overlap with: replay forward + backward from a CUDA graph
            rc = m.forward_backward_graph(tokens, targets, stream)
            return rc | m.update(lr, beta1, beta2, eps, weight_decay, t, stream)
        rc = m.forward(tokens, targets, stream)
        rc |= m.backward_head(stream)
        if self.exchange.world == 1:
            for l in range(self.L - 1, -1, -1):
                rc |= m.backward_layer(l, stream)
            rc |= m.backward_embedding(stream)
            return rc | m.update(lr, beta1, beta2, eps, weight_decay, t, stream)
        for l in range(self.L - 1, -1, -1):
            rc |= m.backward_layer(l, stream)
            ranges = [self.block[l]] + ([self.lnf] if l == self.L - 1 else [])
            self.exchange.exchange([self._slice(r) for r in ranges], stream, tag=ranges)
        rc |= m.backward_embedding(stream)
        self.exchange.exchange([self._slice(self.embed)], stream, tag=[self.embed])
        while True:
            ranges = self.exchange.wait_next(stream)
            if ranges is None:
                break
            for lo, hi in ranges:
                rc |= m.update_range(lo, hi - lo, lr, beta1, beta2, eps, weight_decay, t, stream)
        return rc

    def _sharded_step(self, tokens, targets, lr, beta1, beta2, eps, weight_decay, t, stream):
        m, sx = self.model, self.sharded
        rc = m.forward(tokens, targets, stream)
        rc |= m.backward_head(stream)
        for l in range(self.L - 1, -1, -1):
            rc |= m.backward_layer(l, stream)
            sx.reduce(*self.block[l], stream=stream)
            if l == self.L - 1:
                sx.reduce(*self.lnf, stream=stream)
        rc |= m.backward_embedding(stream)
        sx.reduce(*self.embed, stream=stream)
        sx.finish(stream)
        for first, count in sx.owned():
            rc |= m.update_range(first, count, lr, beta1, beta2, eps, weight_decay, t, stream)
        sx.gather(stream)
        return rc
