"""A serving loop built from flash_nsa/serving.py on one GPU: requests are admitted into the page pool (two of them share a
prefix), prefilled in one packed batch through NSAAttention, then decoded token by token through CUDA graphs of the decode
step (batch padded to the captured size), while the pool grows their token and compressed-row pages.  Every output row is
compared with the CPU oracle evaluated on the whole un-paged sequence (rows are causal, so row t of the full sequence is
the reference for the step that produced token t)."""
import pytest
import torch

from oracle import nsa_oracle as O

pytestmark = pytest.mark.gpu
TOL = 2e-2


def _oracle(q, k, v, w, cfg):
    L = q.size(0)
    cu = [0, L]
    ck = O.mean_pool(k.float(), cu).bfloat16().float()
    cv = O.mean_pool(v.float(), cu).bfloat16().float()
    cmp_o, lse = O.cmp_attn(q.float(), ck, cv, cu)
    # the serving layer passes the forced-block counts swapped, as the reference's layer does: 2 initial blocks, 1 local
    topk = O.topk_select(O.slc_scores(q.float(), ck, lse, cu), cu, num_init=cfg.num_local_blocks, num_local=cfg.num_init_blocks)
    slc_o, _ = O.slc_attn(q.float(), k.float(), v.float(), topk, cu)
    swa_o, _ = O.swa(q.float(), k.float(), v.float(), cu)
    return O.combine(cmp_o, slc_o, swa_o, w.float())


def test_prefill_then_graph_decode_through_the_serving_pieces():
    from flash_nsa.serving import DecodeGraphs, NSAAttention, NSAServingConfig, PagePool, SequenceState, prepare_decode, prepare_prefill
    QH, KH, D = 16, 4, 128
    cfg = NSAServingConfig(page_size=128, max_model_len=2048)
    dev = torch.device("cuda", torch.cuda.current_device())
    g = torch.Generator().manual_seed(11)
    prompts, steps = [300, 300, 97], 40
    shared = torch.randint(0, 1000, (256,), generator=g).tolist()
    toks = [shared + torch.randint(0, 1000, (44,), generator=g).tolist(), shared + torch.randint(0, 1000, (44,), generator=g).tolist(),
            torch.randint(0, 1000, (97,), generator=g).tolist()]
    lens = [p + steps for p in prompts]
    # activations are a function of (sequence, position); the two sequences with a common prefix get the same K/V there
    mk = lambda *s: torch.randn(*s, generator=g).bfloat16()
    data = [dict(q=mk(L, QH, D), k=mk(L, KH, D), v=mk(L, KH, D), w=mk(L, QH, 3)) for L in lens]
    for name in ("k", "v"):
        data[1][name][:256] = data[0][name][:256]
    refs = [_oracle(d["q"], d["k"], d["v"], d["w"], cfg) for d in data]

    pool = PagePool(48, cfg)
    k_cache = torch.zeros(48, cfg.page_size, KH, D, dtype=torch.bfloat16, device=dev)
    v_cache = torch.zeros_like(k_cache)
    layer = NSAAttention(QH, D, D ** -0.5, KH, cfg)
    layer.bind_cache(k_cache, v_cache)
    seqs = [SequenceState(t, cfg) for t in toks]
    for s in seqs:
        assert pool.can_allocate(s)
        pool.allocate(s)
    assert seqs[1].num_cached_tokens == 256 and seqs[1].block_table[:2] == seqs[0].block_table[:2]

    # ---- prefill of everything that is not cached (sequence 1 only brings its last 44 tokens)
    st = prepare_prefill(seqs, cfg, dev)
    first = [s.num_cached_tokens for s in seqs]
    cat = lambda name: torch.cat([data[i][name][first[i]:prompts[i]] for i in range(3)]).to(dev)
    o = layer(cat("q"), cat("k"), cat("v"), cat("w"), st)
    off = 0
    for i in range(3):
        n = prompts[i] - first[i]
        err = (o[off:off + n].float().cpu() - refs[i][first[i]:prompts[i]]).abs()
        assert err.flatten().kthvalue(int(0.998 * err.numel())).values.item() <= TOL and err.max().item() <= 10 * TOL, f"prefill seq {i}"
        off += n

    # ---- decode through CUDA graphs (3 sequences run in the graph captured for 4)
    graphs = DecodeGraphs(layer, 8, QH, KH, D, cfg, dev)
    assert graphs.batch_sizes == [1, 2, 4, 8]
    for step in range(steps):
        for i, s in enumerate(seqs):
            s.append_token(int(torch.randint(0, 1000, (1,), generator=g)))
            assert pool.can_append(s)
            pool.may_append(s)
        st = prepare_decode(seqs, cfg, dev)
        pos = [len(s) - 1 for s in seqs]
        row = lambda name: torch.stack([data[i][name][pos[i]] for i in range(3)]).to(dev)
        o = graphs.run(row("q"), row("k"), row("v"), row("w"), st)
        for i in range(3):
            err = (o[i].float().cpu() - refs[i][pos[i]]).abs().max().item()
            assert err <= TOL, f"decode step {step} seq {i}: {err}"
    # the compressed rows the loop left in the cache are the pooled rows of the whole sequences
    flat = k_cache.view(-1, KH, D)
    for i, s in enumerate(seqs):
        rows = torch.tensor([s.cmp_block_table[j // cfg.page_size] * cfg.page_size + j % cfg.page_size for j in range(s.cmp_len)], device=dev)
        ref = O.mean_pool(data[i]["k"].float(), [0, lens[i]])
        assert (flat[rows].float().cpu() - ref).abs().max().item() <= 8e-3
    for s in seqs:
        pool.deallocate(s)
    assert not pool.used
