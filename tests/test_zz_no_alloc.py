"""The allocation-free variant of the key-block -> queries index (`nsa_k2q_index_static`).

Some hosts cannot allocate device memory where they call the library (all free memory already belongs to their own
pool, or they are inside a region of their runtime where allocation is forbidden).  For them the library carries its
own small scratch array; this test drives that entry point through the C ABI, twice in a row (the array is shared and
keeps the previous call's contents, which the call itself must clear), and checks it against the ordinary entry point.
Lists are compared as sorted rows: the order inside one list is not fixed by either entry point.

The file name sorts last on purpose, so a run that stops at the first failure has already run every other test.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _sorted_lists(offsets, tokens):
    out = []
    off = offsets.cpu()
    tok = tokens.cpu()
    for kh in range(off.shape[0]):
        rows = []
        for r in range(off.shape[1] - 1):
            rows.append(sorted(tok[kh, off[kh, r]:off[kh, r + 1]].tolist()))
        out.append(rows)
    return out


def test_static_scratch_index_matches_regular_one():
    import flash_nsa  # noqa: F401
    from flash_nsa import NSAHelper, _lib
    from flash_nsa.ops import get_bind_from_find
    from flash_nsa.ops.topk import k2q_index_into
    NSAHelper.reset_context_parallel()
    NSAHelper.set_hyperparameters()
    g = torch.Generator().manual_seed(123)
    for lens in ([700, 130], [257]):        # two calls in a row, different sizes: stale cursors would show
        cu = [0]
        for L in lens:
            cu.append(cu[-1] + L)
        T, KH, top_n = cu[-1], 2, 16
        NSAHelper.init_cu_seqlens(torch.tensor(cu, dtype=torch.int32, device="cuda"))
        # a valid selection: forced blocks first, then distinct random earlier blocks
        topk = torch.full((KH, T, top_n), 99, dtype=torch.int32)
        for b, L in enumerate(lens):
            for t in range(L):
                nk = t // 64
                forced = [0] + [x for x in (nk, nk - 1) if x > 0]
                rest = [x for x in torch.randperm(nk + 1, generator=g).tolist() if x not in forced]
                row = (forced + rest)[:min(top_n, nk + 1)]
                for kh in range(KH):
                    topk[kh, cu[b] + t, :len(row)] = torch.tensor(row, dtype=torch.int32)
        topk = topk.cuda()
        ref_off, ref_tok = get_bind_from_find(topk)
        off = torch.full_like(ref_off, -7)
        tok = torch.full((KH, T * top_n), -7, dtype=torch.int32, device="cuda")
        k2q_index_into(topk, off, tok)
        torch.cuda.synchronize()
        assert torch.equal(off, ref_off)
        assert _sorted_lists(off, tok) == _sorted_lists(ref_off, ref_tok)


def test_static_scratch_rejects_oversize():
    from flash_nsa import _lib
    S = _lib.structs
    p = S["NsaK2qParams"]()
    dummy = torch.zeros(8, dtype=torch.int32, device="cuda")
    p.topk = p.offsets = p.tokens = p.blk_cu = dummy.data_ptr()
    p.meta.piece_cu = dummy.data_ptr()
    p.hp.top_n, p.hp.block_size = 16, 64
    p.KH, p.n_blocks_total, p.Tq = 8, 40000, 1      # 320000 cursor entries > 262144
    with pytest.raises(_lib.NsaError, match="exceeds the built-in scratch"):
        _lib.call("nsa_k2q_index_static", p, torch.cuda.current_stream().cuda_stream)
