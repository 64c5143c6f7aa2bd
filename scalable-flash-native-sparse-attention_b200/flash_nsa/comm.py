"""Context-parallel exchange: all-gather of K/V shards into a full-sequence buffer and reduce-scatter of the
fp32 dK/dV, over a torch.distributed process group (NCCL over NVLink on GPUs).

Same role as the reference's `Comm` (flash_nsa/comm.py:15-68), different mechanics: the gather buffers are
double-buffered so the gather of the next kv-head group is issued BEFORE the current group's kernels and
overlaps them, and the cp_mode=2 zig-zag is undone by an out-of-place reorder kernel into the final buffer.
With CPU tensors (gloo, used by the multi-process host-logic tests) the reorder is done with torch indexing
and the reduce-scatter falls back to all-reduce + slice, since gloo has no reduce-scatter.
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
        self.gather = {key: [torch.empty(n, heads, dd, dtype=dtype, device=device) for _ in range(2)] for key, dd in dims.items()}
        self.turn = {self.KEY: 0, self.VALUE: 0}
        self.pending = {}
        self.ready = {}
        self.grads = None
        if with_grads:
            self.grads = {self.GRAD_KEY: torch.empty(n, heads, d, dtype=torch.float32, device=device),
                          self.GRAD_VALUE: torch.empty(n, heads, vd, dtype=torch.float32, device=device)}
            self.local = {self.GRAD_KEY: torch.empty(t_local, heads, d, dtype=torch.float32, device=device),
                          self.GRAD_VALUE: torch.empty(t_local, heads, vd, dtype=torch.float32, device=device)}
        self.backend = dist.get_backend(process_group)

    # -------------------------------------------------------------- K / V
    @torch.no_grad()
    def all_gather(self, x, key):
        """Start gathering the local shard `x` [t, heads, d]; rank-major order (un-shuffled in wait())."""
        buf = self.gather[key][self.turn[key]]
        self.turn[key] ^= 1
        h = dist.all_gather_into_tensor(buf, x.contiguous(), group=self.pg, async_op=True)
        self.pending[key] = (h, buf)

    @torch.no_grad()
    def wait(self, key):
        """Block the current stream until the pending operation on `key` is done; for K/V returns the full
        sequence [t*W, heads, d] in sequential token order."""
        if key not in self.pending:
            return self.ready.get(key)
        h, buf = self.pending.pop(key)
        h.wait()
        if key in (self.KEY, self.VALUE) and self.cp_mode == 2:
            buf = _reorder(buf, self.W, "unshuffle")
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
        """Zero-filled global fp32 dK, dV for one head group."""
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
        self.pending[key] = (h, out)
        return out
