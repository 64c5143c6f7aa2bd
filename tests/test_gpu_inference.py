"""Paged-KV prefill / chunked prefill / decode against the CPU oracle run on the un-paged sequences
(the reference validates its paged ops the same way: against the training ops on the same tokens)."""
import pytest
import torch

from oracle import nsa_oracle as O

pytestmark = pytest.mark.gpu
TOL = 2e-2
PAGE = 128


class Cache:
    """A toy block manager: token pages and compressed-row pages come from one shuffled free list."""

    def __init__(self, lens, KH, D, seed):
        g = torch.Generator().manual_seed(seed)
        self.lens = lens
        self.y_lens = [max((L - 32) // 16 + 1, 0) for L in lens]
        n_tok = [O.cdiv(L, PAGE) for L in lens]
        n_cmp = [max(O.cdiv(y, PAGE), 1) for y in self.y_lens]
        total = sum(n_tok) + sum(n_cmp) + 3
        free = torch.randperm(total, generator=g).tolist()
        self.k = torch.zeros(total, PAGE, KH, D, dtype=torch.bfloat16)
        self.v = torch.zeros(total, PAGE, KH, D, dtype=torch.bfloat16)
        w1, w2 = max(n_tok), max(n_cmp)
        self.block_tables = torch.full((len(lens), w1), -1, dtype=torch.int32)
        self.cmp_block_tables = torch.full((len(lens), w2), -1, dtype=torch.int32)
        for b in range(len(lens)):
            for i in range(n_tok[b]):
                self.block_tables[b, i] = free.pop()
            for i in range(n_cmp[b]):
                self.cmp_block_tables[b, i] = free.pop()

    def store(self, b, k, v, start=0):
        for i in range(k.size(0)):
            p = start + i
            pg = int(self.block_tables[b, p // PAGE])
            self.k[pg, p % PAGE] = k[i]
            self.v[pg, p % PAGE] = v[i]

    def cmp_slot(self, b, j):
        return int(self.cmp_block_tables[b, j // PAGE]) * PAGE + j % PAGE

    def cuda(self):
        self.k, self.v = self.k.cuda(), self.v.cuda()
        self.block_tables, self.cmp_block_tables = self.block_tables.cuda(), self.cmp_block_tables.cuda()
        return self


def _seqs(lens, QH, KH, D, seed):
    g = torch.Generator().manual_seed(seed)
    out = []
    for L in lens:
        out.append(dict(q=torch.randn(L, QH, D, generator=g).bfloat16(), k=torch.randn(L, KH, D, generator=g).bfloat16(),
                        v=torch.randn(L, KH, D, generator=g).bfloat16(), w=torch.randn(L, QH, 3, generator=g).bfloat16()))
    return out


def _oracle(s, L):
    """oracle output for the first L tokens of one sequence, computed with bf16-rounded pooled rows like the kernels"""
    q, k, v, w = s["q"][:L].float(), s["k"][:L].float(), s["v"][:L].float(), s["w"][:L].float()
    cu = [0, L]
    ck = O.mean_pool(k, cu).bfloat16().float()
    cv = O.mean_pool(v, cu).bfloat16().float()
    cmp_o, lse = O.cmp_attn(q, ck, cv, cu)
    topk = O.topk_select(O.slc_scores(q, ck, lse, cu), cu)
    slc_o, _ = O.slc_attn(q, k, v, topk, cu)
    swa_o, _ = O.swa(q, k, v, cu)
    return O.combine(cmp_o, slc_o, swa_o, w)


def _bulk_ok(got, ref):
    err = (got.float().cpu() - ref).abs().flatten()
    # a flipped near-tie of the selection moves single rows by one low-score block: the bulk is held to TOL, every element
    # to ten times TOL (the config-4 test below feeds the CUDA selection to the oracle and holds every element to TOL)
    return (err.kthvalue(max(1, int(0.998 * err.numel()))).values.item() <= TOL and err.max().item() <= 10 * TOL
            and bool(torch.isfinite(got).all()))


@pytest.mark.parametrize("QH,KH,D", [(8, 2, 64), (16, 4, 128)])
def test_prefill_chunked_prefill_and_decode(QH, KH, D):
    import flash_nsa
    from flash_nsa import nsa_prefill, nsa_decode
    lens = [700, 330, 1025]
    seqs = _seqs(lens, QH, KH, D, seed=3 + D)
    # ------------------------------------------------------------------ 1. one-shot prefill of a prefix
    prefix = [448, 100, 777]
    cache = Cache([L + 4 for L in lens], KH, D, seed=9)
    for b, s in enumerate(seqs):
        cache.store(b, s["k"][:prefix[b]], s["v"][:prefix[b]])
    cache.cuda()

    def prefill(start, end):
        x_len = [e - s_ for s_, e in zip(start, end)]
        x_cu = torch.tensor([0] + torch.tensor(x_len).cumsum(0).tolist(), dtype=torch.int32, device="cuda")
        y_len = [max((e - 32) // 16 + 1, 0) for e in end]
        y_cu = torch.tensor([0] + torch.tensor(y_len).cumsum(0).tolist(), dtype=torch.int32, device="cuda")
        slots = []
        for b in range(len(lens)):
            for j in range(y_len[b]):
                new = 16 * j + 31 >= start[b]          # the window ends inside the new tokens
                slots.append(cache.cmp_slot(b, j) if new else -1)
        q = torch.cat([seqs[b]["q"][start[b]:end[b]] for b in range(len(lens))]).cuda()
        w = torch.cat([seqs[b]["w"][start[b]:end[b]] for b in range(len(lens))]).cuda()
        o = nsa_prefill(q, cache.k, cache.v, w, x_cu, y_cu, max(x_len), max(y_len),
                        torch.tensor(end, dtype=torch.int32, device="cuda"), cache.block_tables,
                        torch.tensor(slots, dtype=torch.int32, device="cuda"), cache.cmp_block_tables)
        return o, x_len

    o, x_len = prefill([0, 0, 0], prefix)
    off = 0
    for b in range(len(lens)):
        assert _bulk_ok(o[off:off + x_len[b]], _oracle(seqs[b], prefix[b])), f"prefill seq {b}"
        off += x_len[b]

    # ------------------------------------------------------------------ 2. chunked prefill of the rest on top of the prefix
    end = [L - 1 for L in lens]
    for b, s in enumerate(seqs):
        cache_cpu_k, cache_cpu_v = s["k"][prefix[b]:end[b]], s["v"][prefix[b]:end[b]]
        for i in range(cache_cpu_k.size(0)):
            p = prefix[b] + i
            pg = int(cache.block_tables[b, p // PAGE])
            cache.k[pg, p % PAGE] = cache_cpu_k[i].cuda()
            cache.v[pg, p % PAGE] = cache_cpu_v[i].cuda()
    o, x_len = prefill(prefix, end)
    off = 0
    for b in range(len(lens)):
        ref = _oracle(seqs[b], end[b])[prefix[b]:]
        assert _bulk_ok(o[off:off + x_len[b]], ref), f"chunked prefill seq {b}"
        off += x_len[b]

    # ------------------------------------------------------------------ 3. decode the last token (+ one padding row)
    for b, s in enumerate(seqs):
        p = lens[b] - 1
        pg = int(cache.block_tables[b, p // PAGE])
        cache.k[pg, p % PAGE] = s["k"][p].cuda()
        cache.v[pg, p % PAGE] = s["v"][p].cuda()
    ctx = lens + [0]
    slot = []
    for b, L in enumerate(lens):
        has_new = (L % 16 == 0) and L >= 32
        slot.append(cache.cmp_slot(b, (L - 32) // 16) if has_new else -1)
    slot.append(-1)
    pad = lambda t: torch.cat([t, torch.full((1, t.size(1)), -1, dtype=torch.int32, device="cuda")])
    q = torch.stack([seqs[b]["q"][lens[b] - 1] for b in range(len(lens))] + [torch.zeros(QH, D).bfloat16()]).cuda()
    w = torch.stack([seqs[b]["w"][lens[b] - 1] for b in range(len(lens))] + [torch.zeros(QH, 3).bfloat16()]).cuda()
    from flash_nsa.inference import nsa_decode_unfused, nsa_decode_fused
    args = (q, cache.k, cache.v, w, torch.tensor(ctx, dtype=torch.int32, device="cuda"), pad(cache.block_tables),
            torch.tensor(slot, dtype=torch.int32, device="cuda"), pad(cache.cmp_block_tables))
    o_unfused = nsa_decode_unfused(*args)
    o, tk = nsa_decode_fused(*args, return_topk=True)
    assert torch.equal(o, nsa_decode(*args))           # the public entry point takes the fused path here
    assert (o.float() - o_unfused.float()).abs().max().item() <= TOL
    for b in range(len(lens)):                         # slot layout of the selection: forced blocks first
        nkb = (lens[b] - 1) // 64
        row = tk[0, b].tolist()
        nv = min(16, nkb + 1)
        assert row[0] == 0 and row[1] == nkb and row[2] == nkb - 1 and max(row) <= nkb
        assert len(set(row[:nv])) == nv and min(row[:nv]) >= 0 and all(x == -1 for x in row[nv:])
    assert tk[:, -1].eq(-1).all()
    for b in range(len(lens)):
        ref = _oracle(seqs[b], lens[b])[-1:]
        assert (o[b:b + 1].float().cpu() - ref).abs().max().item() <= TOL, f"decode seq {b}"
    assert float(o[-1].float().abs().max()) == 0.0      # padding row: no tokens -> zeros


@pytest.mark.parametrize("QH,KH,D", [(32, 1, 128), (64, 2, 64), (24, 1, 64)])
def test_more_than_16_query_heads_per_kv_head_on_the_paged_path(QH, KH, D):
    """The reference loops groups of min(G, 16) heads in its paged kernels; here the scorer sums the groups' probabilities
    before the pooling, the attention kernels run the groups as separate tiles, and nsa_decode takes the op-by-op path."""
    from flash_nsa import nsa_prefill, nsa_decode
    lens = [520, 203]
    seqs = _seqs(lens, QH, KH, D, seed=21 + QH)
    B = len(lens)
    cache = Cache([L + 1 for L in lens], KH, D, seed=6)
    for b, s in enumerate(seqs):
        cache.store(b, s["k"][:lens[b] - 1], s["v"][:lens[b] - 1])
    cache.cuda()
    end = [L - 1 for L in lens]
    y_len = [max((e - 32) // 16 + 1, 0) for e in end]
    x_cu = torch.tensor([0, end[0], end[0] + end[1]], dtype=torch.int32, device="cuda")
    y_cu = torch.tensor([0, y_len[0], y_len[0] + y_len[1]], dtype=torch.int32, device="cuda")
    slots = torch.tensor([cache.cmp_slot(b, j) for b in range(B) for j in range(y_len[b])], dtype=torch.int32, device="cuda")
    q = torch.cat([seqs[b]["q"][:end[b]] for b in range(B)]).cuda()
    w = torch.cat([seqs[b]["w"][:end[b]] for b in range(B)]).cuda()
    o = nsa_prefill(q, cache.k, cache.v, w, x_cu, y_cu, max(end), max(y_len), torch.tensor(end, dtype=torch.int32, device="cuda"),
                    cache.block_tables, slots, cache.cmp_block_tables)
    off = 0
    for b in range(B):
        assert _bulk_ok(o[off:off + end[b]], _oracle(seqs[b], end[b])), f"prefill seq {b}"
        off += end[b]
    # decode the last token of every sequence
    for b, s in enumerate(seqs):
        p = lens[b] - 1
        pg = int(cache.block_tables[b, p // PAGE])
        cache.k[pg, p % PAGE] = s["k"][p].cuda()
        cache.v[pg, p % PAGE] = s["v"][p].cuda()
    slot = [cache.cmp_slot(b, (L - 32) // 16) if (L % 16 == 0 and L >= 32) else -1 for b, L in enumerate(lens)]
    qd = torch.stack([seqs[b]["q"][lens[b] - 1] for b in range(B)]).cuda()
    wd = torch.stack([seqs[b]["w"][lens[b] - 1] for b in range(B)]).cuda()
    od = nsa_decode(qd, cache.k, cache.v, wd, torch.tensor(lens, dtype=torch.int32, device="cuda"), cache.block_tables,
                    torch.tensor(slot, dtype=torch.int32, device="cuda"), cache.cmp_block_tables)
    for b in range(B):
        ref = _oracle(seqs[b], lens[b])[-1:]
        assert (od[b:b + 1].float().cpu() - ref).abs().max().item() <= TOL, f"decode seq {b}"


def test_decode_long_contexts_use_the_round_based_selection():
    """Above 256 selection blocks (16K tokens) the one-launch decode step selects by rounds of warp-wide arg-max instead of
    rank counting: same list as the op-by-op path (which runs the scoring kernel of prefill), same output."""
    from flash_nsa.inference import nsa_decode_unfused, nsa_decode_fused
    QH, KH, D = 8, 2, 64
    lens = [20000, 16500, 3000]
    B = len(lens)
    g = torch.Generator().manual_seed(77)
    cache = Cache(lens, KH, D, seed=8)
    flat_k = cache.k.view(-1, KH, D)
    flat_v = cache.v.view(-1, KH, D)
    for b, L in enumerate(lens):
        pos = torch.arange(L)
        rows = cache.block_tables[b].long()[pos // PAGE] * PAGE + pos % PAGE
        flat_k[rows] = torch.randn(L, KH, D, generator=g).bfloat16()
        flat_v[rows] = torch.randn(L, KH, D, generator=g).bfloat16()
    cache.cuda()
    from flash_nsa.inference import mean_pooling_prefill
    y_len = [(L - 32) // 16 + 1 for L in lens]
    y_cu = torch.tensor([0] + torch.tensor(y_len).cumsum(0).tolist(), dtype=torch.int32, device="cuda")
    slots = torch.tensor([cache.cmp_slot(b, j) for b in range(B) for j in range(y_len[b])], dtype=torch.int32, device="cuda")
    for c in (cache.k, cache.v):
        mean_pooling_prefill(c, y_cu, max(y_len), slot_mapping=slots, block_table=cache.block_tables)
    q = torch.randn(B, QH, D, generator=g).bfloat16().cuda()
    w = torch.randn(B, QH, 3, generator=g).bfloat16().cuda()
    args = (q, cache.k, cache.v, w, torch.tensor(lens, dtype=torch.int32, device="cuda"), cache.block_tables,
            torch.full((B,), -1, dtype=torch.int32, device="cuda"), cache.cmp_block_tables)
    o_ref = nsa_decode_unfused(*args)
    o, tk = nsa_decode_fused(*args, return_topk=True)
    assert (o.float() - o_ref.float()).abs().max().item() <= TOL
    for b, L in enumerate(lens):
        nkb = (L - 1) // 64
        for h in range(KH):
            row = tk[h, b].tolist()
            assert row[0] == 0 and row[1] == nkb and row[2] == nkb - 1
            assert len(set(row)) == 16 and min(row) >= 0 and max(row) <= nkb


def _cluster_case(lens, KH, G, D, seed, want=None):
    """One fused decode step on a page table as wide as a 64K-token context needs (few sequences then run as clusters)
    against the same sequences many times over (enough CTAs for one each) and against the op-by-op path."""
    from flash_nsa.inference import nsa_decode_unfused, nsa_decode_fused, mean_pooling_prefill
    from flash_nsa.inference.ops import decode_cluster_size
    B, QH = len(lens), KH * G
    g = torch.Generator().manual_seed(seed)
    cache = Cache(lens, KH, D, seed=seed)
    flat_k = cache.k.view(-1, KH, D)
    flat_v = cache.v.view(-1, KH, D)
    for b, L in enumerate(lens):
        pos = torch.arange(L)
        rows = cache.block_tables[b].long()[pos // PAGE] * PAGE + pos % PAGE
        flat_k[rows] = torch.randn(L, KH, D, generator=g).bfloat16()
        flat_v[rows] = torch.randn(L, KH, D, generator=g).bfloat16()
    cache.cuda()
    y_old = [max((L - 1 - 32) // 16 + 1, 0) for L in lens]             # the rows earlier steps have written
    y_cu = torch.tensor([0] + torch.tensor(y_old).cumsum(0).tolist(), dtype=torch.int32, device="cuda")
    slots = torch.tensor([cache.cmp_slot(b, j) for b in range(B) for j in range(y_old[b])], dtype=torch.int32, device="cuda")
    if slots.numel():
        for c in (cache.k, cache.v):
            mean_pooling_prefill(c, y_cu, max(y_old), slot_mapping=slots, block_table=cache.block_tables)
    new_slot = [cache.cmp_slot(b, (L - 32) // 16) if (L % 16 == 0 and L >= 32) else -1 for b, L in enumerate(lens)]
    wide = torch.zeros(B, 65536 // PAGE, dtype=torch.int32, device="cuda")
    wide[:, :cache.block_tables.size(1)] = cache.block_tables
    q = torch.randn(B, QH, D, generator=g).bfloat16().cuda()
    w = torch.randn(B, QH, 3, generator=g).bfloat16().cuda()
    args = (q, cache.k, cache.v, w, torch.tensor(lens, dtype=torch.int32, device="cuda"), wide,
            torch.tensor(new_slot, dtype=torch.int32, device="cuda"), cache.cmp_block_tables)
    cs = decode_cluster_size(B, KH, PAGE, wide.stride(0), D=D)
    assert cs == want if want is not None else cs > 1
    # the same sequences many times over fill the GPU by themselves: one CTA per (sequence, kv head)
    rep = 148 // (B * KH) + 1
    assert decode_cluster_size(B * rep, KH, PAGE, wide.stride(0), D=D) == 1
    o_ref, tk_ref = nsa_decode_fused(*[a.repeat(rep, *([1] * (a.dim() - 1))) if i in (0, 3, 4, 5, 6, 7) else a for i, a in enumerate(args)],
                                     return_topk=True)
    o_ref, tk_ref = o_ref[:B], tk_ref[:, :B]
    written = [s_ for s_ in new_slot if s_ >= 0]
    fk, fv = cache.k.view(-1, KH, D), cache.v.view(-1, KH, D)
    rows_ref = (fk[written].clone(), fv[written].clone())
    fk[written] = 0
    fv[written] = 0
    o, tk = nsa_decode_fused(*args, return_topk=True)
    assert torch.equal(fk[written], rows_ref[0]) and torch.equal(fv[written], rows_ref[1])
    assert not written or bool((rows_ref[0] != 0).any())
    o_un = nsa_decode_unfused(*args)
    assert torch.equal(tk.sort(-1).values, tk_ref.sort(-1).values)
    assert (o.float() - o_ref.float()).abs().max().item() <= 4e-3      # bf16 rounding of a different merge order
    assert (o.float() - o_un.float()).abs().max().item() <= TOL


@pytest.mark.parametrize("B,KH,want", [(1, 2, 8), (5, 4, 4), (16, 4, 2)])
def test_decode_of_few_sequences_splits_each_over_a_cluster(B, KH, want):
    """With few sequences and a page table wide enough for long contexts the one-launch decode step runs as clusters of
    `want` CTAs per (sequence, kv head), each taking every want-th tile.  Same selection, output and new compressed row as
    with one CTA each and as the op-by-op path, for contexts that leave some CTAs of a cluster without a compressed tile,
    with a tile each, and with many."""
    lens = ([9008, 48, 700, 2500, 4100, 64, 1, 5008] * 2)[:B]          # multiples of 16 complete a compressed row
    _cluster_case(lens, KH, 4, 128, seed=500 + B, want=want)


@pytest.mark.parametrize("seed", range(8))
def test_cluster_decode_on_random_shapes(seed):
    """Random batch sizes, head counts, head dims and context lengths (1 to 6000 tokens, some completing a compressed row)
    through the cluster form of the decode step."""
    import random
    rng = random.Random(9000 + seed)
    KH = rng.choice([1, 2, 4])
    G = rng.choice([1, 2, 4, 8, 16])
    D = rng.choice([64, 128])
    B = rng.randint(1, max(1, 16 // KH))
    lens = [rng.choice([rng.randint(1, 6000), 16 * rng.randint(2, 370)]) for _ in range(B)]
    _cluster_case(lens, KH, G, D, seed=9000 + seed)


def test_rows_past_a_sequence_end_may_hold_anything():
    """Never-written cache memory (here: NaN everywhere a row was not stored) must not reach a result: the tile kernels read
    whole tiles of a page, and a zero probability times NaN is NaN."""
    from flash_nsa import nsa_prefill, nsa_decode
    from flash_nsa.inference import nsa_decode_unfused
    QH, KH, D = 16, 4, 128
    lens = [333, 1000, 70]
    seqs = _seqs(lens, QH, KH, D, seed=31)
    B = len(lens)
    cache = Cache(lens, KH, D, seed=12)
    cache.k.fill_(float("nan"))
    cache.v.fill_(float("nan"))
    end = [L - 1 for L in lens]
    for b, s in enumerate(seqs):
        cache.store(b, s["k"][:end[b]], s["v"][:end[b]])
    cache.cuda()
    y_len = [max((e - 32) // 16 + 1, 0) for e in end]
    x_cu = torch.tensor([0] + torch.tensor(end).cumsum(0).tolist(), dtype=torch.int32, device="cuda")
    y_cu = torch.tensor([0] + torch.tensor(y_len).cumsum(0).tolist(), dtype=torch.int32, device="cuda")
    slots = torch.tensor([cache.cmp_slot(b, j) for b in range(B) for j in range(y_len[b])], dtype=torch.int32, device="cuda")
    q = torch.cat([seqs[b]["q"][:end[b]] for b in range(B)]).cuda()
    w = torch.cat([seqs[b]["w"][:end[b]] for b in range(B)]).cuda()
    o = nsa_prefill(q, cache.k, cache.v, w, x_cu, y_cu, max(end), max(y_len), torch.tensor(end, dtype=torch.int32, device="cuda"),
                    cache.block_tables, slots, cache.cmp_block_tables)
    assert bool(torch.isfinite(o).all())
    off = 0
    for b in range(B):
        assert _bulk_ok(o[off:off + end[b]], _oracle(seqs[b], end[b])), f"prefill seq {b}"
        off += end[b]
    for b, s in enumerate(seqs):
        p = lens[b] - 1
        pg = int(cache.block_tables[b, p // PAGE])
        cache.k[pg, p % PAGE] = s["k"][p].cuda()
        cache.v[pg, p % PAGE] = s["v"][p].cuda()
    slot = [cache.cmp_slot(b, (L - 32) // 16) if (L % 16 == 0 and L >= 32) else -1 for b, L in enumerate(lens)]
    qd = torch.stack([seqs[b]["q"][lens[b] - 1] for b in range(B)]).cuda()
    wd = torch.stack([seqs[b]["w"][lens[b] - 1] for b in range(B)]).cuda()
    args = (qd, cache.k, cache.v, wd, torch.tensor(lens, dtype=torch.int32, device="cuda"), cache.block_tables,
            torch.tensor(slot, dtype=torch.int32, device="cuda"), cache.cmp_block_tables)
    for fn in (nsa_decode, nsa_decode_unfused):
        od = fn(*args)
        assert bool(torch.isfinite(od).all()), fn.__name__
        for b in range(B):
            ref = _oracle(seqs[b], lens[b])[-1:]
            assert (od[b:b + 1].float().cpu() - ref).abs().max().item() <= TOL, f"{fn.__name__} seq {b}"


def test_decode_of_very_short_contexts():
    """The first tokens of a sequence: no compressed row yet (context < 32), the first one (32), a single selection block,
    the first block boundary (64, 65): one fused decode step each, against the oracle."""
    from flash_nsa import nsa_decode
    QH, KH, D = 16, 4, 128
    lens = [1, 2, 31, 32, 33, 63, 64, 65, 128, 129]
    B = len(lens)
    seqs = _seqs(lens, QH, KH, D, seed=91)
    cache = Cache(lens, KH, D, seed=13)
    for b, s_ in enumerate(seqs):
        cache.store(b, s_["k"], s_["v"])
    cache.cuda()
    # the compressed rows that earlier steps would have written: all but the one this step completes
    from flash_nsa.inference import mean_pooling_prefill
    y_old = [max((L - 1 - 32) // 16 + 1, 0) for L in lens]
    y_cu = torch.tensor([0] + torch.tensor(y_old).cumsum(0).tolist(), dtype=torch.int32, device="cuda")
    slots_old = torch.tensor([cache.cmp_slot(b, j) for b in range(B) for j in range(y_old[b])], dtype=torch.int32, device="cuda")
    if slots_old.numel():
        for c in (cache.k, cache.v):
            mean_pooling_prefill(c, y_cu, max(y_old), slot_mapping=slots_old, block_table=cache.block_tables)
    slot = [cache.cmp_slot(b, (L - 32) // 16) if (L % 16 == 0 and L >= 32) else -1 for b, L in enumerate(lens)]
    qd = torch.stack([seqs[b]["q"][lens[b] - 1] for b in range(B)]).cuda()
    wd = torch.stack([seqs[b]["w"][lens[b] - 1] for b in range(B)]).cuda()
    od = nsa_decode(qd, cache.k, cache.v, wd, torch.tensor(lens, dtype=torch.int32, device="cuda"), cache.block_tables,
                    torch.tensor(slot, dtype=torch.int32, device="cuda"), cache.cmp_block_tables)
    assert bool(torch.isfinite(od).all())
    for b in range(B):
        ref = _oracle(seqs[b], lens[b])[-1:]
        assert (od[b:b + 1].float().cpu() - ref).abs().max().item() <= TOL, f"context {lens[b]}"


def test_decode_writes_the_new_compressed_row():
    from flash_nsa.inference import kv_mean_pooling_decode
    KH, D = 2, 64
    L = 160                                   # multiple of 16: the decode step completes compressed row (160-32)/16 = 8
    s = _seqs([L], 4, KH, D, seed=5)[0]
    cache = Cache([L], KH, D, seed=1)
    cache.store(0, s["k"], s["v"])
    cache.cuda()
    slot = cache.cmp_slot(0, 8)
    kv_mean_pooling_decode(cache.k, cache.v, torch.tensor([slot], dtype=torch.int32, device="cuda"), cache.block_tables,
                           torch.tensor([L], dtype=torch.int32, device="cuda"))
    ref_k = O.mean_pool(s["k"].float(), [0, L])[8]
    ref_v = O.mean_pool(s["v"].float(), [0, L])[8]
    got_k = cache.k.view(-1, KH, D)[slot].float().cpu()
    got_v = cache.v.view(-1, KH, D)[slot].float().cpu()
    assert (got_k - ref_k).abs().max().item() <= 8e-3 and (got_v - ref_v).abs().max().item() <= 8e-3


def test_generation_loop_prefill_then_many_decode_steps():
    """A serving loop: prefill a prompt, then 70 decode steps (crossing 16-token pooling boundaries, 64-token selection
    blocks and a page boundary).  Every step stores the new K/V rows with store_kvcache, passes the slot of the compressed
    row that the step completes, and is compared with the oracle run on the whole un-paged prefix; at the end the
    compressed rows held by the cache equal the pooled rows of the whole sequence."""
    from flash_nsa import nsa_prefill, nsa_decode
    from flash_nsa.inference import store_kvcache
    QH, KH, D = 16, 4, 128
    prompt, steps = [200, 77], 70
    lens = [p + steps for p in prompt]
    seqs = _seqs(lens, QH, KH, D, seed=9)
    cache = Cache(lens, KH, D, seed=4).cuda()
    B = len(lens)

    def tok_slot(b, pos):
        return int(cache.block_tables[b, pos // PAGE]) * PAGE + pos % PAGE

    # ---- prefill of the prompts (K/V rows go in through store_kvcache)
    k_new = torch.cat([seqs[b]["k"][:prompt[b]] for b in range(B)]).cuda()
    v_new = torch.cat([seqs[b]["v"][:prompt[b]] for b in range(B)]).cuda()
    slots = torch.tensor([tok_slot(b, p) for b in range(B) for p in range(prompt[b])], dtype=torch.int32, device="cuda")
    store_kvcache(k_new, v_new, cache.k, cache.v, slots)
    y_len = [max((p - 32) // 16 + 1, 0) for p in prompt]
    x_cu = torch.tensor([0, prompt[0], prompt[0] + prompt[1]], dtype=torch.int32, device="cuda")
    y_cu = torch.tensor([0, y_len[0], y_len[0] + y_len[1]], dtype=torch.int32, device="cuda")
    cmp_slots = torch.tensor([cache.cmp_slot(b, j) for b in range(B) for j in range(y_len[b])], dtype=torch.int32, device="cuda")
    q = torch.cat([seqs[b]["q"][:prompt[b]] for b in range(B)]).cuda()
    w = torch.cat([seqs[b]["w"][:prompt[b]] for b in range(B)]).cuda()
    o = nsa_prefill(q, cache.k, cache.v, w, x_cu, y_cu, max(prompt), max(y_len), torch.tensor(prompt, dtype=torch.int32, device="cuda"),
                    cache.block_tables, cmp_slots, cache.cmp_block_tables)
    off = 0
    for b in range(B):
        assert _bulk_ok(o[off:off + prompt[b]], _oracle(seqs[b], prompt[b])), f"prefill seq {b}"
        off += prompt[b]

    # ---- decode steps
    refs = [_oracle(seqs[b], lens[b]) for b in range(B)]      # causal: row t only depends on the first t+1 tokens
    worst = 0.0
    for s in range(steps):
        ctx = [prompt[b] + s + 1 for b in range(B)]           # tokens in the cache after this step's store
        pos = [c - 1 for c in ctx]
        k1 = torch.stack([seqs[b]["k"][pos[b]] for b in range(B)]).cuda()
        v1 = torch.stack([seqs[b]["v"][pos[b]] for b in range(B)]).cuda()
        store_kvcache(k1, v1, cache.k, cache.v, torch.tensor([tok_slot(b, pos[b]) for b in range(B)], dtype=torch.int32, device="cuda"))
        slot = [cache.cmp_slot(b, (c - 32) // 16) if (c % 16 == 0 and c >= 32) else -1 for b, c in enumerate(ctx)]
        q1 = torch.stack([seqs[b]["q"][pos[b]] for b in range(B)]).cuda()
        w1 = torch.stack([seqs[b]["w"][pos[b]] for b in range(B)]).cuda()
        o1 = nsa_decode(q1, cache.k, cache.v, w1, torch.tensor(ctx, dtype=torch.int32, device="cuda"), cache.block_tables,
                        torch.tensor(slot, dtype=torch.int32, device="cuda"), cache.cmp_block_tables)
        for b in range(B):
            err = (o1[b].float().cpu() - refs[b][pos[b]]).abs().max().item()
            worst = max(worst, err)
            assert err <= TOL, f"decode step {s} seq {b}: {err}"
    # ---- the cache's compressed rows are the pooled rows of the whole sequences
    for b in range(B):
        Y = (lens[b] - 32) // 16 + 1
        ref_k = O.mean_pool(seqs[b]["k"].float(), [0, lens[b]])
        got = torch.stack([cache.k.view(-1, KH, D)[cache.cmp_slot(b, j)] for j in range(Y)]).float().cpu()
        assert (got - ref_k).abs().max().item() <= 8e-3


def test_baseline_config4_paged_decode_and_chunked_prefill():
    """BASELINE config 4 at its full shape, exactly as the benchmark builds it (32 q heads / 8 kv heads / d = 128, page
    256, randomly permuted page table, 64 decode sequences with contexts U[4096, 8192], and a 2048-token chunk on a
    6144-token prefix): for EVERY decode sequence the output row, the selected blocks (as sets, near-ties by the oracle's
    scores) and the compressed row the step writes, and for 64 sampled rows of the chunk the prefill output, the
    selection and the pooled rows it writes, against the oracle evaluated on the un-paged sequences.  Paged = un-paged
    and chunked = one-shot are the identities the reference checks in inference.ipynb (cells 34, 43, 50)."""
    from bench import Config4
    c4 = Config4(torch.device("cuda", torch.cuda.current_device()))
    o, tk = c4.decode(return_topk=True)
    res = c4.check_decode(o, tk)                  # all 64 sequences
    assert res["max_err"] <= TOL
    assert res["near_tie_rows"] <= 8, res         # of 64 x 8 rows
    assert torch.equal(o, c4.decode())            # public entry point, same result when the step is repeated
    res = c4.check_prefill(c4.prefill(), n_rows=64)
    assert res["max_err"] <= TOL and res["rows"] >= 64
    # the paged entry points reach contexts where all 16 slots are used and most blocks are NOT selected
    assert min(c4.ctx) >= 4096 and all((L - 1) // 64 + 1 >= 64 for L in c4.ctx)
