"""Host logic of the serving-side pieces (flash_nsa/serving.py) on CPU: page accounting of the pool (token pages shared by
prefix, compressed-row pages private), admission / growth rules, and the per-step tensors: token slots, the lengths and
slots of the compressed rows in a prefill, and the slot of the row a decode step completes."""
import random

import torch

from flash_nsa.serving import NSAServingConfig, PagePool, SequenceState, prepare_decode, prepare_prefill


def _cfg(page=16):
    return NSAServingConfig(page_size=page, kernel_size=8, stride=4, block_size=8, max_model_len=4096)


def test_sequence_lengths_follow_the_compression_rule():
    cfg = _cfg()
    for n in (0, 7, 8, 11, 12, 100, 256, 257):
        s = SequenceState(list(range(n)), cfg)
        assert s.cmp_len == max((n - 8) // 4 + 1, 0)
        assert s.num_blocks == -(-n // 16) and s.num_cmp_blocks == -(-s.cmp_len // 16)
        if n:
            assert s.last_block_num_tokens == n - (s.num_blocks - 1) * 16


def test_pool_shares_prefix_pages_but_not_compressed_pages():
    cfg = _cfg()
    pool = PagePool(64, cfg)
    a = SequenceState(list(range(100)), cfg)          # 6 full token pages + 1 partial; cmp_len 24 -> 2 pages
    assert pool.can_allocate(a)
    pool.allocate(a)
    assert len(a.block_table) == 7 and len(a.cmp_block_table) == 2 and a.num_cached_tokens == 0
    b = SequenceState(list(range(64)) + [7] * 40, cfg)   # same first 4 pages
    pool.allocate(b)
    assert b.num_cached_tokens == 64 and b.block_table[:4] == a.block_table[:4]
    assert not set(b.block_table[4:]) & set(a.block_table)
    assert not set(b.cmp_block_table) & set(a.cmp_block_table)         # compressed rows are never shared
    used = len(pool.used)
    assert used == 7 + 2 + (len(b.block_table) - 4) + len(b.cmp_block_table)
    pool.deallocate(a)
    assert all(pool.ref[p] == 1 for p in b.block_table)                # shared pages survive their first owner
    pool.deallocate(b)
    assert len(pool.free) == 64 and not pool.used
    # a freed full page is still found by content
    c = SequenceState(list(range(100)), cfg)
    pool.allocate(c)
    assert c.num_cached_tokens == 96


def test_pool_growth_allocates_token_and_compressed_pages_when_they_are_needed():
    cfg = _cfg()
    pool = PagePool(40, cfg)
    s = SequenceState(list(range(5)), cfg)
    pool.allocate(s)
    assert len(s.block_table) == 1 and s.cmp_block_table == []
    rng = random.Random(0)
    for _ in range(300):
        s.append_token(rng.randrange(1000))
        assert pool.can_append(s)
        pool.may_append(s)
        assert len(s.block_table) == s.num_blocks and len(s.cmp_block_table) == s.num_cmp_blocks
    assert len(set(s.block_table) | set(s.cmp_block_table)) == s.num_blocks + s.num_cmp_blocks
    small = PagePool(2, cfg)
    t = SequenceState(list(range(16)), cfg)
    small.allocate(t)
    t.append_token(1)
    assert not small.can_append(t)


def test_prefill_and_decode_step_tensors():
    cfg = _cfg()
    pool = PagePool(64, cfg)
    a, b = SequenceState(list(range(37)), cfg), SequenceState(list(range(100, 120)), cfg)
    pool.allocate(a)
    pool.allocate(b)
    st = prepare_prefill([a, b], cfg, device="cpu")
    assert st.cu_seqlens_q.tolist() == [0, 37, 57] and st.max_seqlen_q == 37 and st.context_lens.tolist() == [37, 20]
    assert st.positions.tolist() == list(range(37)) + list(range(20))
    want = [a.block_table[p // 16] * 16 + p % 16 for p in range(37)] + [b.block_table[p // 16] * 16 + p % 16 for p in range(20)]
    assert st.slot_mapping.tolist() == want
    assert st.cmp_cu_seqlens.tolist() == [0, a.cmp_len, a.cmp_len + b.cmp_len] and st.cmp_max_seqlen == max(a.cmp_len, b.cmp_len)
    want = [s.cmp_block_table[j // 16] * 16 + j % 16 for s in (a, b) for j in range(s.cmp_len)]
    assert st.cmp_slot_mapping.tolist() == want
    assert st.block_tables.shape == (2, 3) and st.block_tables[1, 2].item() == -1
    # decode: the row completed when the length reaches a multiple of the stride, including the first row of a new page
    for _ in range(80):
        for s in (a, b):
            s.append_token(5)
            pool.may_append(s)
        st = prepare_decode([a, b], cfg, device="cpu")
        for i, s in enumerate((a, b)):
            n = len(s)
            assert st.context_lens[i].item() == n and st.positions[i].item() == n - 1
            assert st.slot_mapping[i].item() == s.block_table[(n - 1) // 16] * 16 + (n - 1) % 16
            if n % 4 == 0 and n >= 8:
                j = (n - 8) // 4
                assert st.cmp_slot_mapping[i].item() == s.cmp_block_table[j // 16] * 16 + j % 16
            else:
                assert st.cmp_slot_mapping[i].item() == -1


def test_index_ranges_follow_the_cell_size():
    """Host-side rule of the selected backward's index: a range as long as it takes for a (range, block) cell to hold 128 rows,
    at least 4096 rows, none once that needs more than 32 MiB of q per range (long sequences under context parallelism)."""
    from flash_nsa.ops.topk import backward_index_sizes
    G, D = 16, 128
    assert backward_index_sizes(G, D, 65536, 1024) == (8192, 512)        # 64K tokens on one GPU
    assert backward_index_sizes(G, D, 32768, 512) == (4096, 512)
    assert backward_index_sizes(G, D, 131072, 2048)[0] == 0              # 128K tokens: cells of 128 rows would need 16K-row ranges
    assert backward_index_sizes(G, D, 131072, 16384)[0] == 0             # one shard of 8 at 1M tokens
    assert backward_index_sizes(G, D, 23888, 118) == (4096, 512)         # packed short sequences: the floor of 4096 rows
    assert backward_index_sizes(G, D, 2048, 32)[0] == 0                  # fewer rows than one range
    assert backward_index_sizes(4, 64, 65536, 1024)[1] == 64 * 32        # 32 tokens per query tile at G = 4
