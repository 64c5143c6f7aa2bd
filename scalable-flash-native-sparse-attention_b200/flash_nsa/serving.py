"""Engine-side pieces a paged-KV serving loop needs around `nsa_prefill` / `nsa_decode`.

The reference ships these inside its nano-vllm fork (nano-vllm/nanovllm/engine/{sequence,block_manager,model_runner}.py
and layers/attention.py); this module provides the same pieces for the attention path alone, free of the model, the
scheduler and the sampler:

  SequenceState      lengths and page lists of one request: token pages and, separately, pages for its compressed rows
                     (sequence.py:66-92)
  PagePool           the page allocator: prefix-cached token pages, never-shared compressed-row pages, allocate / append /
                     free with the reference's admission rules (block_manager.py:59-141)
  prepare_prefill    per-step tensors of a (chunked) prefill batch: packed lengths, token slots, block tables, and the
                     compressed-row lengths / slots / tables (model_runner.py:186-259)
  prepare_decode     the same for one decode step, including the slot of the compressed row a sequence completes when its
                     length reaches a multiple of the stride (model_runner.py:261-290)
  NSAAttention       the attention layer's call: store the new K/V rows, then nsa_prefill or nsa_decode on the caches
                     (layers/attention.py:26-118, 184-221)
  DecodeGraphs       CUDA graphs of the decode step for a ladder of batch sizes, replayed on padded static inputs
                     (model_runner.py:292-368)

Everything here is host logic plus copies into static buffers; the kernels are the ones behind nsa_prefill / nsa_decode.
"""
import hashlib
from collections import deque
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from .inference import nsa_decode, nsa_prefill, store_kvcache


@dataclass
class NSAServingConfig:
    """Constants of the attention path of a served model (the reference keeps them in a global "constant context")."""
    page_size: int = 256
    kernel_size: int = 32
    stride: int = 16
    block_size: int = 64
    top_n: int = 16
    num_init_blocks: int = 1
    num_local_blocks: int = 2
    window_size: int = 512
    fixed_y_maxlen: int = 8192
    fixed_num_slc_blocks: int = 2048
    cmp_num_splits: int = 0
    slc_num_splits: int = 0
    max_model_len: int = 131072


class SequenceState:
    """One request: its tokens and the pages that hold its K/V rows and its compressed rows."""
    _ids = 0

    def __init__(self, token_ids: Sequence[int], cfg: NSAServingConfig):
        SequenceState._ids += 1
        self.seq_id = SequenceState._ids
        self.cfg = cfg
        self.token_ids = list(token_ids)
        self.num_prompt_tokens = len(self.token_ids)
        self.num_cached_tokens = 0          # leading tokens whose K/V pages were found in the prefix cache
        self.block_table: List[int] = []
        self.cmp_block_table: List[int] = []

    def __len__(self):
        return len(self.token_ids)

    @property
    def num_blocks(self):
        return -(-len(self) // self.cfg.page_size)

    @property
    def num_cached_blocks(self):
        return self.num_cached_tokens // self.cfg.page_size

    @property
    def last_block_num_tokens(self):
        return len(self) - (self.num_blocks - 1) * self.cfg.page_size

    @property
    def cmp_len(self):
        """Compressed rows the sequence has: windows of kernel_size tokens every stride tokens that are complete."""
        return max((len(self) - self.cfg.kernel_size) // self.cfg.stride + 1, 0)

    @property
    def num_cmp_blocks(self):
        return -(-self.cmp_len // self.cfg.page_size)

    def block(self, i):
        return self.token_ids[i * self.cfg.page_size:(i + 1) * self.cfg.page_size]

    def append_token(self, token_id: int):
        self.token_ids.append(token_id)


class PagePool:
    """Page allocator over `num_pages` cache pages.  Full token pages are content-hashed (chained with the hash of the
    page before) and shared between sequences with the same prefix; compressed-row pages are private to their sequence and
    come from the same pool, so admission counts both kinds."""

    def __init__(self, num_pages: int, cfg: NSAServingConfig):
        self.cfg = cfg
        self.ref = [0] * num_pages
        self.hash_of = [-1] * num_pages
        self.tokens_of: List[Optional[list]] = [None] * num_pages
        self.by_hash: Dict[int, int] = {}
        self.free = deque(range(num_pages))
        self.used = set()

    @staticmethod
    def page_hash(token_ids, prefix=-1):
        h = hashlib.blake2b(digest_size=8)
        if prefix != -1:
            h.update(int(prefix).to_bytes(8, "little"))
        h.update(np.asarray(token_ids, dtype=np.int64).tobytes())
        return int.from_bytes(h.digest(), "little")

    def _take(self, page=None):
        page = self.free[0] if page is None else page
        assert self.ref[page] == 0
        self.free.remove(page)
        self.used.add(page)
        self.ref[page], self.hash_of[page], self.tokens_of[page] = 1, -1, None
        return page

    def _release(self, page):
        self.ref[page] -= 1
        if self.ref[page] == 0:
            self.used.remove(page)
            self.free.append(page)

    # -- admission of a new sequence
    def can_allocate(self, seq: SequenceState) -> bool:
        return len(self.free) >= seq.num_blocks + seq.num_cmp_blocks

    def allocate(self, seq: SequenceState):
        assert not seq.block_table and not seq.cmp_block_table
        h, miss = -1, False
        page_size = self.cfg.page_size
        for i in range(seq.num_blocks):
            toks = seq.block(i)
            h = self.page_hash(toks, h) if len(toks) == page_size else -1
            page = self.by_hash.get(h, -1) if h != -1 else -1
            if page == -1 or self.tokens_of[page] != toks:
                miss = True                      # from the first miss on, every later page is new
            if miss:
                page = self._take()
            else:
                seq.num_cached_tokens += page_size
                if page in self.used:
                    self.ref[page] += 1
                else:
                    self._take(page)
            if h != -1:
                self.hash_of[page], self.tokens_of[page] = h, toks
                self.by_hash[h] = page
            seq.block_table.append(page)
        for _ in range(seq.num_cmp_blocks):      # compressed rows are not shared between sequences
            seq.cmp_block_table.append(self._take())

    def deallocate(self, seq: SequenceState):
        for page in reversed(seq.block_table):
            self._release(page)
        for page in reversed(seq.cmp_block_table):
            self._release(page)
        seq.num_cached_tokens = 0
        seq.block_table.clear()
        seq.cmp_block_table.clear()

    # -- growth by one token (call after SequenceState.append_token)
    def can_append(self, seq: SequenceState) -> bool:
        page_size = self.cfg.page_size
        need = int(len(seq) % page_size == 1) + int(seq.num_cmp_blocks > len(seq.cmp_block_table))
        return len(self.free) >= need

    def may_append(self, seq: SequenceState):
        page_size = self.cfg.page_size
        if len(seq) % page_size == 1 or not seq.block_table:
            seq.block_table.append(self._take())
        elif len(seq) % page_size == 0:          # the last page just became full: it can be shared from now on
            last = seq.block_table[-1]
            prefix = self.hash_of[seq.block_table[-2]] if len(seq.block_table) > 1 else -1
            toks = seq.block(seq.num_blocks - 1)
            h = self.page_hash(toks, prefix)
            self.hash_of[last], self.tokens_of[last] = h, toks
            self.by_hash[h] = last
        if seq.num_cmp_blocks > len(seq.cmp_block_table):
            seq.cmp_block_table.append(self._take())


# ------------------------------------------------------------------------------------------------ per-step tensors
@dataclass
class StepInputs:
    is_prefill: bool
    positions: torch.Tensor                 # [t] int64 position of every new token
    slot_mapping: torch.Tensor              # [t] int32 flat cache row of every new token
    context_lens: torch.Tensor              # [b] int32 tokens in the cache after this step's store
    block_tables: torch.Tensor              # [b, w] int32, -1 padded
    cmp_slot_mapping: torch.Tensor          # prefill: one entry per compressed row of the batch; decode: [b], -1 = none
    cmp_block_tables: torch.Tensor          # [b, w2] int32, -1 padded
    cu_seqlens_q: Optional[torch.Tensor] = None     # prefill: [b+1] int32 offsets of the new tokens
    max_seqlen_q: int = 0
    cmp_cu_seqlens: Optional[torch.Tensor] = None   # prefill: [b+1] int32 offsets of the compressed rows
    cmp_max_seqlen: int = 0


def _dev(values, dtype, device):
    t = torch.tensor(values, dtype=dtype)
    if torch.device(device).type == "cuda":
        return t.pin_memory().to(device, non_blocking=True)
    return t


def _tables(lists, device):
    width = max(max((len(x) for x in lists), default=1), 1)
    return _dev([list(x) + [-1] * (width - len(x)) for x in lists], torch.int32, device)


def prepare_prefill(seqs: List[SequenceState], cfg: NSAServingConfig, device="cuda") -> StepInputs:
    """Inputs of a prefill step over the tokens of every sequence that are not in the prefix cache.  Every compressed row of
    a sequence gets its slot: rows whose window lies in the cached prefix are simply pooled again (as the reference does)."""
    positions, slots, ctx, cu_q, cmp_cu, cmp_slots = [], [], [], [0], [0], []
    max_q = cmp_max = 0
    page = cfg.page_size
    for s in seqs:
        n, first = len(s), s.num_cached_tokens
        ctx.append(n)
        positions.extend(range(first, n))
        cu_q.append(cu_q[-1] + n - first)
        max_q = max(max_q, n - first)
        for i in range(s.num_cached_blocks, s.num_blocks):
            start = s.block_table[i] * page
            rows = page if i != s.num_blocks - 1 else s.last_block_num_tokens
            slots.extend(range(start, start + rows))
        cmp_cu.append(cmp_cu[-1] + s.cmp_len)
        cmp_max = max(cmp_max, s.cmp_len)
        for i in range(s.num_cmp_blocks):
            start = s.cmp_block_table[i] * page
            cmp_slots.extend(range(start, start + min(page, s.cmp_len - i * page)))
    return StepInputs(True, _dev(positions, torch.int64, device), _dev(slots, torch.int32, device), _dev(ctx, torch.int32, device),
                      _tables([s.block_table for s in seqs], device), _dev(cmp_slots, torch.int32, device),
                      _tables([s.cmp_block_table for s in seqs], device), _dev(cu_q, torch.int32, device), max_q,
                      _dev(cmp_cu, torch.int32, device), cmp_max)


def prepare_decode(seqs: List[SequenceState], cfg: NSAServingConfig, device="cuda") -> StepInputs:
    """Inputs of one decode step (every sequence already holds its newest token).  A sequence whose length is a multiple
    of the stride completes compressed row cmp_len - 1 in this step: its slot is row (cmp_len - 1) % page of the last
    compressed-row page."""
    page = cfg.page_size
    positions, slots, ctx, cmp_slots = [], [], [], []
    for s in seqs:
        n = len(s)
        positions.append(n - 1)
        ctx.append(n)
        slots.append(s.block_table[-1] * page + s.last_block_num_tokens - 1)
        c = s.cmp_len
        cmp_slots.append(s.cmp_block_table[-1] * page + (c - 1) % page if (n % cfg.stride == 0 and c > 0) else -1)
    return StepInputs(False, _dev(positions, torch.int64, device), _dev(slots, torch.int32, device), _dev(ctx, torch.int32, device),
                      _tables([s.block_table for s in seqs], device), _dev(cmp_slots, torch.int32, device),
                      _tables([s.cmp_block_table for s in seqs], device))


# ------------------------------------------------------------------------------------------------ the attention layer's call
class NSAAttention(torch.nn.Module):
    """The attention call of a served layer: q [t,qh,d], k/v [t,kh,d] of the step's new tokens and gate logits w [t,qh,3]
    -> o [t,qh,d].  The caches are [pages, page_size, kh, d]; `forward` writes the new rows, then runs the prefill or the
    decode entry point on the caches.  The forced-block counts are passed the way the reference's layer passes them: its
    `num_local_blocks` as the number of initial blocks and its `num_init_blocks` as the number of local ones
    (nano-vllm/nanovllm/layers/attention.py:68-69, 113-114)."""

    def __init__(self, num_heads, head_dim, scale, num_kv_heads, cfg: NSAServingConfig):
        super().__init__()
        self.num_heads, self.head_dim, self.scale, self.num_kv_heads, self.cfg = num_heads, head_dim, scale, num_kv_heads, cfg
        self.k_cache = self.v_cache = torch.tensor([])

    def bind_cache(self, k_cache, v_cache):
        assert k_cache.dim() == 4 and k_cache.size(1) == self.cfg.page_size and k_cache.shape == v_cache.shape
        self.k_cache, self.v_cache = k_cache, v_cache

    def forward(self, q, k, v, w, step: StepInputs):
        c = self.cfg
        store_kvcache(k, v, self.k_cache, self.v_cache, step.slot_mapping)
        common = dict(kernel_size=c.kernel_size, stride=c.stride, block_size=c.block_size, top_n=c.top_n,
                      num_init_blocks=c.num_local_blocks, num_local_blocks=c.num_init_blocks, window_size=c.window_size,
                      fixed_y_maxlen=c.fixed_y_maxlen, fixed_num_slc_blocks=c.fixed_num_slc_blocks, sm_scale=self.scale)
        if step.is_prefill:
            return nsa_prefill(q, self.k_cache, self.v_cache, w, x_cu_seqlens=step.cu_seqlens_q, y_cu_seqlens=step.cmp_cu_seqlens,
                               x_maxlen=step.max_seqlen_q, y_maxlen=step.cmp_max_seqlen, context_lens=step.context_lens,
                               block_tables=step.block_tables, cmp_slot_mapping=step.cmp_slot_mapping,
                               cmp_block_tables=step.cmp_block_tables, **common)
        return nsa_decode(q, self.k_cache, self.v_cache, w, context_lens=step.context_lens, block_tables=step.block_tables,
                          cmp_slot_mapping=step.cmp_slot_mapping, cmp_block_tables=step.cmp_block_tables,
                          cmp_num_splits=c.cmp_num_splits, slc_num_splits=c.slc_num_splits, **common)


# ------------------------------------------------------------------------------------------------ CUDA graphs of the decode step
class DecodeGraphs:
    """CUDA graphs of `fn(q, k, v, w, step) -> o` (a decode step: one new token per sequence) for batch sizes 1, 2, 4, 8, 16,
    32, ... up to `max_bs`, captured once on static buffers.  `run` copies a real batch into the smallest graph that holds
    it, pads the rest (context length 0 and slot -1: the kernels write nothing and return zeros for those rows) and replays.
    All captures share one memory pool, largest batch first."""

    def __init__(self, fn, max_bs, num_heads, num_kv_heads, head_dim, cfg: NSAServingConfig, device="cuda", dtype=torch.bfloat16):
        self.fn, self.cfg = fn, cfg
        max_bs = min(max_bs, 512)
        max_pages = -(-cfg.max_model_len // cfg.page_size)
        max_cmp = max((cfg.max_model_len - cfg.kernel_size) // cfg.stride + 1, 1)
        max_cmp_pages = -(-max_cmp // cfg.page_size)
        z = lambda *shape, dt=torch.int32: torch.zeros(*shape, dtype=dt, device=device)
        self.vars = dict(q=z(max_bs, num_heads, head_dim, dt=dtype), k=z(max_bs, num_kv_heads, head_dim, dt=dtype),
                         v=z(max_bs, num_kv_heads, head_dim, dt=dtype), w=z(max_bs, num_heads, 3, dt=dtype),
                         positions=z(max_bs, dt=torch.int64), slot_mapping=z(max_bs), context_lens=z(max_bs),
                         block_tables=z(max_bs, max_pages), cmp_slot_mapping=z(max_bs), cmp_block_tables=z(max_bs, max_cmp_pages),
                         out=z(max_bs, num_heads, head_dim, dt=dtype))
        self.vars["slot_mapping"].fill_(-1)
        self.vars["cmp_slot_mapping"].fill_(-1)
        self.batch_sizes = [b for b in (1, 2, 4, 8) if b <= max_bs] + list(range(16, max_bs + 1, 16))
        self.graphs, self.pool = {}, None
        V = self.vars
        for bs in reversed(self.batch_sizes):
            step = StepInputs(False, V["positions"][:bs], V["slot_mapping"][:bs], V["context_lens"][:bs], V["block_tables"][:bs],
                              V["cmp_slot_mapping"][:bs], V["cmp_block_tables"][:bs])
            args = (V["q"][:bs], V["k"][:bs], V["v"][:bs], V["w"][:bs], step)
            V["out"][:bs] = fn(*args)                       # warm-up outside the capture (first-call set-up, allocations)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, self.pool):
                V["out"][:bs] = fn(*args)
            if self.pool is None:
                self.pool = g.pool()
            self.graphs[bs] = g
        torch.cuda.synchronize()

    def run(self, q, k, v, w, step: StepInputs):
        bs = q.size(0)
        gbs = next(b for b in self.batch_sizes if b >= bs)
        V = self.vars
        for name, t in (("q", q), ("k", k), ("v", v), ("w", w), ("positions", step.positions)):
            V[name][:bs] = t
        V["slot_mapping"].fill_(-1)
        V["slot_mapping"][:bs] = step.slot_mapping
        V["context_lens"].zero_()
        V["context_lens"][:bs] = step.context_lens
        V["block_tables"][:bs, :step.block_tables.size(1)] = step.block_tables
        V["cmp_slot_mapping"].fill_(-1)
        V["cmp_slot_mapping"][:bs] = step.cmp_slot_mapping
        V["cmp_block_tables"][:bs, :step.cmp_block_tables.size(1)] = step.cmp_block_tables
        self.graphs[gbs].replay()
        return V["out"][:bs]
