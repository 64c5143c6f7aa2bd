"""Context-parallel exchange: all-gather of K/V shards into a full-sequence buffer and reduce-scatter of the
fp32 dK/dV, over a torch.distributed process group (NCCL over NVLink on GPUs).

Same role as the reference's `Comm` (flash_nsa/comm.py:15-68), different mechanics.  The full-sequence K/V
buffers are double-buffered, so the caller issues the gather of kv-head group h+1 right after it has waited
for group h, BEFORE group h's attention kernels are enqueued: a NCCL collective starts once the work that was
on the compute stream at the time of the call has finished, so issued there it runs under those kernels.  For
cp_mode=2 the gather lands rank-major in a staging buffer and an out-of-place reorder kernel un-zig-zags it
into the final buffer on a side stream, also under the kernels; `wait()` only makes the compute stream wait
for that stream's event.  With CPU tensors (gloo, used by the multi-process host-logic tests) the reorder is
done with torch indexing and the reduce-scatter falls back to all-reduce + slice, since gloo has no
reduce-scatter.
"""
import torch
import torch.distributed as dist


def _reorder(x, world_size, mode):
    if x.is_cuda:
        from .ops.reorder import reorder
        return reorder(x, world_size, shuffle_mode=mode)
    chunks = list(x.chunk(2 * world_size))
    if mode == "shuffle":
        out = []
        for i in range(world_size):
            out += [chunks[i], chunks[2 * world_size - 1 - i]]
        return torch.cat(out, 0)
    return torch.cat(chunks[::2] + chunks[1::2][::-1], 0)


class Comm:
    KEY = "k"
    VALUE = "v"
    GRAD_KEY = "dk"
    GRAD_VALUE = "dv"

    def __init__(self, process_group, t_local, world_size, heads, d, vd, dtype, device, cp_mode=1, with_grads=False):
        assert cp_mode in (1, 2)
        self.pg, self.W, self.cp_mode = process_group, world_size, cp_mode
        self.t, self.heads = t_local, heads
        dims = {self.KEY: d, self.VALUE: vd}
        n = t_local * world_size
        # final (sequential token order) buffers, two per key; cp_mode 2 gathers into one staging buffer per key first
        self.final = {key: [torch.empty(n, heads, dd, dtype=dtype, device=device) for _ in range(2)] for key, dd in dims.items()}
        self.stage = ({key: torch.empty(n, heads, dd, dtype=dtype, device=device) for key, dd in dims.items()}
                      if cp_mode == 2 else None)
        self.turn = {self.KEY: 0, self.VALUE: 0}
        self.pending = {}
        self.ready = {}
        self.grads = None
        self.cuda = torch.device(device).type == "cuda"
        self.side = torch.cuda.Stream(device=device) if (self.cuda and cp_mode == 2) else None
        if with_grads:
            self.grads = {self.GRAD_KEY: torch.empty(n, heads, d, dtype=torch.float32, device=device),
                          self.GRAD_VALUE: torch.empty(n, heads, vd, dtype=torch.float32, device=device)}
            self.local = {self.GRAD_KEY: torch.empty(t_local, heads, d, dtype=torch.float32, device=device),
                          self.GRAD_VALUE: torch.empty(t_local, heads, vd, dtype=torch.float32, device=device)}
        self.backend = dist.get_backend(process_group)

    # -------------------------------------------------------------- K / V
    @torch.no_grad()
    def all_gather(self, x, key):
        """Start gathering the local shard `x` [t, heads, d] into the buffer that the PREVIOUS wait(key) did not return.
        Safe to call while kernels that read the other buffer are still queued on the compute stream."""
        out = self.final[key][self.turn[key]]
        self.turn[key] ^= 1
        src = x.contiguous()
        if self.cp_mode == 1:
            h = dist.all_gather_into_tensor(out, src, group=self.pg, async_op=True)
            self.pending[key] = (h, out, None, src)
            return
        stage = self.stage[key]
        h = dist.all_gather_into_tensor(stage, src, group=self.pg, async_op=True)
        if self.side is None:                       # CPU tensors
            h.wait()
            out.copy_(_reorder(stage, self.W, "unshuffle"))
            self.pending[key] = (None, out, None, None)
            return
        # un-zig-zag on the side stream as soon as the gather is done; the staging buffer is free for the next gather by
        # then because that gather is issued after wait(key), i.e. after the compute stream took this event
        with torch.cuda.stream(self.side):
            h.wait()
            from .ops.reorder import reorder
            reorder(stage, self.W, shuffle_mode="unshuffle", out=out)
            ev = torch.cuda.Event()
            ev.record(self.side)
        # `src` (a packed copy of the shard when the head slice is strided) was allocated on the compute stream and is read by
        # the collective on another one: it is kept until wait(key), i.e. until the compute stream has waited for this event.
        # (h.wait() above releases the collective's own hold on it, and the allocator would hand the block out again.)
        self.pending[key] = (None, out, ev, src)

    @torch.no_grad()
    def wait(self, key):
        """Make the current stream wait for the pending operation on `key`; for K/V returns the full sequence
        [t*W, heads, d] in sequential token order."""
        if key not in self.pending:
            return self.ready.get(key)
        h, buf, ev, src = self.pending.pop(key)
        if h is not None:
            h.wait()
        if ev is not None:
            torch.cuda.current_stream().wait_event(ev)
        del src
        self.ready[key] = buf
        return buf

    def wait_all(self):
        for key in list(self.pending):
            self.wait(key)

    def release(self):
        """The gathered K/V of the current head group will not be read by launches issued after this call."""
        self.ready.pop(self.KEY, None)
        self.ready.pop(self.VALUE, None)

    # -------------------------------------------------------------- dK / dV
    def grad_buffers(self):
        """Zero-filled global fp32 dK, dV for one head group.  The zero fill is ordered behind the previous group's
        reduce-scatter, which reads the same tensors (cp_mode 1) or their shuffled copies (cp_mode 2): callers wait for
        GRAD_KEY / GRAD_VALUE of a group before asking for the next group's buffers, and this method checks it."""
        assert self.GRAD_KEY not in self.pending and self.GRAD_VALUE not in self.pending, \
            "wait(GRAD_KEY) / wait(GRAD_VALUE) of the previous head group must come before grad_buffers()"
        dk, dv = self.grads[self.GRAD_KEY], self.grads[self.GRAD_VALUE]
        dk.zero_()
        dv.zero_()
        return dk, dv

    @torch.no_grad()
    def reduce_scatter(self, key):
        """Sum the global gradient buffer over ranks and keep this rank's shard; returns the local fp32
        tensor [t, heads, d], valid after wait(key)."""
        full = self.grads[key]
        if self.cp_mode == 2:
            full = _reorder(full, self.W, "shuffle")
        out = self.local[key]
        if self.backend == "gloo":
            h = dist.all_reduce(full, group=self.pg, async_op=True)
            h.wait()
            r = dist.get_rank(self.pg)
            out.copy_(full[r * self.t:(r + 1) * self.t])
            return out
        h = dist.reduce_scatter_tensor(out, full, group=self.pg, async_op=True)
        self.pending[key] = (h, out, None, None)
        return out
