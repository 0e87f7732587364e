"""Host-side launch plans of the few-token products: every K range is covered once, in whole 32-element chunks,
within what the kernels' shared memory takes (no GPU needed)."""
import pytest


@pytest.mark.parametrize("n,k", [(1536, 1536), (1536, 8960), (2048, 1536), (17920, 1536), (151936, 1536), (3584, 18944),
                                 (5120, 13824), (64, 32), (80, 96), (300, 12288), (7, 64)])
def test_k_ranges_cover_the_product(n, k):
    from microllm_rocm_b200.kernels import gemm_bf16
    splits, per = gemm_bf16.gemv_splits(n, k)
    assert splits >= 1 and per % 32 == 0 and (splits - 1) * per < k <= splits * per
    assert per * 2 * 16 <= 160 * 1024                      # sixteen staged token rows fit shared memory
    plan = gemm_bf16.gemv_split_plan(n, k)
    if plan is not None:
        splits, per = plan
        assert splits >= 1 and per % 32 == 0 and (splits - 1) * per < k <= splits * per
        assert per <= gemm_bf16.GEMV_FUSED_MAX_K
        assert -(-n // 16) <= gemm_bf16.GEMV_SPLIT_MAX_TILES
    else:
        assert -(-n // 16) > gemm_bf16.GEMV_SPLIT_MAX_TILES


def test_token_tiles_and_routing_limits():
    from microllm_rocm_b200.kernels import gemm_bf16
    assert [gemm_bf16.token_tile(m) for m in (1, 16, 17, 64, 65, 128, 129, 5000)] == [16, 16, 32, 64, 128, 128, 256, 256]
    assert gemm_bf16.token_tile(5000, dual=True) == 128
    assert gemm_bf16.GEMV_ROUTE_MAX_TOKENS <= gemm_bf16.GEMV_MAX_TOKENS
    assert gemm_bf16.GEMV_SILU_MAX_TOKENS <= gemm_bf16.GEMV_MAX_TOKENS


def test_decode_key_split_grows_with_the_context_and_fits_one_wave():
    from microllm_rocm_b200.kernels import attention
    for items in (1, 2, 16, 128, 400):
        last = 0
        for context in (1, 48, 64, 113, 241, 497, 1009, 4000, 100000):
            splits = attention.decode_splits(items, context)
            assert splits >= max(1, last) or splits == last            # never fewer CTAs for a longer context
            assert splits == 1 or (items * splits <= 2 * attention.SM_COUNT and -(-context // 16) >= 4 * splits)
            last = splits
    assert attention.decode_splits(16, 16) == 1 and attention.decode_splits(16, 2048) == 8
    assert attention.decode_splits(2, 32768) == 16 and attention.decode_splits(128, 2048) == 2


class _Ctx:
    def __init__(self, extras):
        self.extras = extras


def test_a_frozen_decode_plan_is_recognised_as_stale():
    from microllm_rocm_b200.kernels import attention
    key = ("attention_mma", 6, 2, True)
    plan = (None, 8, 1, attention.decode_splits(16, 20), None, 0)       # planned at a context of 20 tokens: one CTA
    ctx = _Ctx({key: plan, ("rope_table", 1): object(), "other": 3})
    assert not attention.decode_plan_stale(ctx, 40)
    assert attention.decode_plan_stale(ctx, 2048)
    attention.forget_plans(ctx)
    assert key not in ctx.extras and len(ctx.extras) == 2 and not attention.decode_plan_stale(ctx, 2048)
