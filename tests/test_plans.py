"""Host-side launch plans of the few-token products: every K range is covered once, in whole 32-element chunks,
within what the kernels' shared memory takes (no GPU needed)."""
import pytest

from microllm_rocm_b200.kernels.device import DEFAULT_SM_COUNT


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
        assert -(-n // 16) <= gemm_bf16.GEMV_SPLIT_MAX_TILES_PER_SM * DEFAULT_SM_COUNT
    else:
        assert -(-n // 16) > gemm_bf16.GEMV_SPLIT_MAX_TILES_PER_SM * DEFAULT_SM_COUNT
    # the tcgen05 streaming product: whole 64-element blocks of K, no empty range, at most one CTA per SM and tile
    for sms in (DEFAULT_SM_COUNT, 132, 16):
        s = gemm_bf16.stream_splits(n, k, sms)
        blocks = -(-k // 64)
        per = -(-blocks // s)
        assert 1 <= s <= gemm_bf16.STREAM_MAX_SPLITS and (s - 1) * per < blocks <= s * per
        assert s == 1 or (s * -(-n // 128) <= sms and per >= gemm_bf16.STREAM_MIN_K_BLOCKS_PER_SPLIT - 1)


def test_plans_follow_the_device_they_are_made_for():
    """A part with fewer multiprocessors gets fewer CTAs per product and smaller clusters per sequence."""
    from microllm_rocm_b200.kernels import attention, gemm_bf16
    assert gemm_bf16.gemv_splits(1536, 8960, 148)[0] > gemm_bf16.gemv_splits(1536, 8960, 32)[0]
    assert gemm_bf16.stream_splits(1536, 8960, 148) > gemm_bf16.stream_splits(1536, 8960, 24)
    assert attention.decode_splits(16, 2048, 148) == 8 and attention.decode_splits(16, 2048, 60) == 4


def test_routing_limits():
    from microllm_rocm_b200.kernels import gemm_bf16
    assert gemm_bf16.GEMV_ROUTE_MAX_TOKENS <= gemm_bf16.GEMV_MAX_TOKENS
    assert gemm_bf16.GEMV_SILU_MAX_TOKENS <= gemm_bf16.GEMV_MAX_TOKENS
    assert gemm_bf16.GEMV_ROUTE_MAX_TOKENS < gemm_bf16.STREAM_MAX_TOKENS < gemm_bf16.PAIR_MIN_TOKENS


def test_decode_key_split_grows_with_the_context_and_fits_one_wave():
    from microllm_rocm_b200.kernels import attention
    for items in (1, 2, 16, 128, 400):
        last = 0
        for context in (1, 48, 64, 113, 241, 497, 1009, 4000, 100000):
            splits = attention.decode_splits(items, context)
            assert splits >= max(1, last) or splits == last            # never fewer CTAs for a longer context
            assert splits == 1 or (items * splits <= 2 * DEFAULT_SM_COUNT and -(-context // 16) >= 4 * splits)
            last = splits
    assert attention.decode_splits(16, 16) == 1 and attention.decode_splits(16, 2048) == 8
    assert attention.decode_splits(2, 32768) == 16 and attention.decode_splits(128, 2048) == 2


def test_the_key_ring_is_for_long_streams_on_a_full_gpu():
    from microllm_rocm_b200.kernels import attention
    assert attention.decode_ring_pays(128, 2, 2073)             # batch 64, two kv heads, clusters of 2: 1,036 keys per CTA
    assert not attention.decode_ring_pays(64, 4, 2073)          # batch 32: 518 keys per CTA
    assert not attention.decode_ring_pays(16, 8, 2073)          # batch 8: fewer CTAs than multiprocessors
    assert attention.decode_ring_pays(64, 4, 8192) and not attention.decode_ring_pays(2, 16, 32768)
    # beside the few-token mma.sync products the next kernel needs the shared memory to start early
    assert not attention.decode_ring_pays(64, 4, 8192, beside_mma_products=True) and attention.decode_ring_pays(128, 2, 8192)


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


def test_captured_batch_sizes():
    from microllm_rocm_b200.engine.decode_graph import BATCH_SIZES, captured_batch
    assert [captured_batch(n, 256) for n in (1, 2, 3, 5, 8, 9, 13, 33, 64, 65, 200, 257, 300)] == \
        [1, 2, 4, 8, 8, 12, 16, 48, 64, 96, 256, 257, 300]
    assert captured_batch(5, 6) == 6 and captured_batch(6, 6) == 6 and captured_batch(3, 3) == 3      # never more rows than request slots... but never fewer than the requests
    assert list(BATCH_SIZES) == sorted(BATCH_SIZES)
