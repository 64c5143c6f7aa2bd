"""This build against the reference's own Triton kernels on the same GPU and inputs (o and every gradient of NSACore on two
packed sequences of 4096 tokens in all, 64 q heads / 4 kv heads / d = 128).  The reference package is the pip-installed copy
under baseline/_ref (git-ignored; it travels with the repository to the GPU box); each side runs in a process of its own
because both packages are called flash_nsa.  Skips where that copy is absent or its kernels do not compile or run."""
import pytest

pytestmark = pytest.mark.gpu


def test_core_matches_the_reference_kernels():
    import reference_gpu_compare as R
    res = R.compare()
    if "unavailable" in res:
        pytest.skip(res["unavailable"])
    # selections: both kernels round the block scores to half precision (p^3), so near-ties at the end of a list can fall
    # either way (measured: 0.6-0.9 % of the rows differ, by one swapped block; the reference's own kernel disagrees with its
    # fp32 torch code on a similar share of rows)
    tk = res["topk"]
    assert tk["fraction"] <= 0.03 and tk["largest_symmetric_difference"] <= 6, tk
    for name in ("o", "dq", "dk", "dv", "dw"):
        r = res[name]
        # two bf16 implementations, each within 2e-2 * max(1, max|x|) of the fp32 oracle, with unordered fp32 / bf16 adds on
        # both sides and selections that may differ in a near-tie: the bulk is held to that bound against each other as well
        # (measured over several runs: at most 1.2e-5 of the elements beyond it, the largest difference 0.06 of max|ref|)
        assert r["frac_over_2e-2"] <= 1e-3, (name, r)
        assert r["max_abs_diff"] <= 0.15 * max(1.0, r["max_abs_ref"]), (name, r)


def test_paged_prefill_and_decode_match_the_reference_kernels():
    """nsa_prefill of three prompts and one nsa_decode step over the same paged caches (pages of 256 rows: the reference's
    window branch over a paged cache needs that), against the reference's inference kernels."""
    import reference_gpu_compare as R
    res = R.compare_inference()
    if "unavailable" in res:
        pytest.skip(res["unavailable"])
    for name in ("prefill", "decode"):
        r = res[name]
        assert r["frac_over_2e-2"] <= 1e-3, (name, r)
        assert r["max_abs_diff"] <= 0.15 * max(1.0, r["max_abs_ref"]), (name, r)

