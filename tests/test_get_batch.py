"""Host logic of the context-parallel batch split (no GPU): shard layout and the cp_mode rule."""
import sys
import os

import torch

from oracle import nsa_oracle as O

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "scalable-flash-native-sparse-attention_b200"))


def _gb():
    import importlib.util
    here = os.path.dirname(os.path.abspath(__file__))
    path = os.path.join(here, "..", "scalable-flash-native-sparse-attention_b200", "flash_nsa", "get_batch.py")
    spec = importlib.util.spec_from_file_location("nsa_get_batch", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_split_matches_the_oracle_shard_ranges():
    gb = _gb()
    T = 64 * 12
    x = torch.arange(T)[None]
    for W in (2, 3, 4):
        for mode in (1, 2):
            for r in range(W):
                got = gb.split_for_cp_rank(x, W, r, mode)[0]
                meta = O.cp_metadata([0, T], r, W, mode)
                want = O.cp_local_slice(torch.arange(T), meta["ranges"])
                assert torch.equal(got, want), (W, mode, r)


def test_cp_mode_rule():
    gb = _gb()
    # one long sequence: longest >= 1.5 x tokens per rank -> zig-zag
    assert gb.get_cp_mode_from_cu_seqlens([0, 8192], 4) == 2
    # many short ones -> contiguous
    assert gb.get_cp_mode_from_cu_seqlens([0, 1000, 2000, 3000, 4000, 5000, 6000, 7000, 8192], 4) == 1
    # exactly at the threshold (1.5 * 2048 = 3072) -> zig-zag
    assert gb.get_cp_mode_from_cu_seqlens([0, 3072, 8192 - 3000, 8192], 4) == 2
    assert gb.get_cp_mode_from_cu_seqlens([0, 3071, 6000, 8192], 4) == 1
    assert gb.get_cp_mode_from_cu_seqlens([0, 100, 8192], 4, threshold=10000) == 1


def test_batch_dict_is_split_in_place():
    gb = _gb()
    T = 256
    batch = {"input_ids": torch.arange(T)[None], "labels": torch.arange(T)[None] + 1, "position_ids": torch.arange(T)[None],
             "cu_seqlens": torch.tensor([0, T], dtype=torch.int32), "other": 7}
    out = gb.get_batch_on_this_cp_rank_for_nsa(dict(batch), cp_size=2, cp_rank=1)
    assert out["cp_mode"] == 2 and out["other"] == 7
    want = torch.cat([torch.arange(64, 128), torch.arange(128, 192)])[None]
    assert torch.equal(out["input_ids"], want) and torch.equal(out["labels"], want + 1)
    same = gb.get_batch_on_this_cp_rank_for_nsa(dict(batch), cp_size=1, cp_rank=0)
    assert torch.equal(same["input_ids"], batch["input_ids"]) and "cp_mode" not in same
