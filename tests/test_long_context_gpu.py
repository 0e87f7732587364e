"""The attention kernels and the engine at the sizes the benchmark runs: prompt portions of 2,048 and 8,192
tokens through the tcgen05 kernel, a later portion that starts thousands of tokens into its sequence, decode
steps at contexts of 2,073 to 16,500 tokens with thread-block clusters of 16, 8 and 2 CTAs per (sequence, kv
head), and two layers of the 1.5B shape against the plain implementation.

At these lengths random inputs hide faults: the softmax of thousands of unit-variance scores is nearly flat,
every output is a mean of thousands of values (about 0.01 in size) and an absolute tolerance passes anything.
So the queries are scaled until a few dozen keys carry the weight, half of the heads get a planted key far back
that must dominate, and errors are measured against the size of the expected row.

The reference here is the formula of `tests/plain` (src/ops/ops.cpp:2343-2384: scale after the dot product,
causal range, softmax, probabilities times values) evaluated for chosen rows in float64 with plain tensor
operations; `test_reference_rows_are_the_plain_formula` holds it against the plain loop itself."""
import math
import os

import numpy as np
import pytest
import torch

from tests.plain import qwen2_plain as plain

DEV = "cuda"
gpu = pytest.mark.gpu


# ------------------------------------------------------------------------------ reference for chosen rows
def reference_rows(q_rows, row_pos, k, v, window):
    """q_rows [R, NH, D] sit at absolute positions row_pos [R] of one sequence with keys k, v [n, NKV, D].
    Returns [R, NH, D] float64."""
    R, NH, D = q_rows.shape
    n, NKV, _ = k.shape
    group = NH // NKV
    q64, k64, v64 = q_rows.double(), k.double(), v.double()
    kh = k64.repeat_interleave(group, dim=1)                   # [n, NH, D]: head h uses kv head h // group
    vh = v64.repeat_interleave(group, dim=1)
    s = torch.einsum("rhd,nhd->rhn", q64, kh) * (1.0 / math.sqrt(float(D)))
    j = torch.arange(n, device=q_rows.device)[None, :]
    pos = row_pos.to(q_rows.device)[:, None]
    visible = j <= pos
    if window is not None:
        visible &= j >= pos - window + 1
    s = s.masked_fill(~visible[:, None, :], float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.einsum("rhn,nhd->rhd", p, vh)


def test_reference_rows_are_the_plain_formula():
    torch.manual_seed(0)
    n, nh, nkv, d = 75, 6, 2, 16
    q, k, v = torch.randn(n, nh, d) * 2, torch.randn(n, nkv, d), torch.randn(n, nkv, d)
    for window in (None, 20):
        want = plain.causal_gqa_attention(q, k, v, window)
        rows = torch.tensor([0, 1, 19, 20, 21, 74])
        got = reference_rows(q[rows], rows, k, v, window)
        assert torch.allclose(got.float(), want[rows], atol=1e-5)


# ------------------------------------------------------------------------------ a paged cache made on the device
class PagedCase:
    """Sequences of the given lengths in a cache of shuffled pages, keys and values drawn on the device in
    bf16; `dense(s)` gathers sequence s back for the reference."""

    def __init__(self, lens, nkv, d, page_size, seed):
        gen = torch.Generator(device=DEV).manual_seed(seed)
        self.lens, self.page_size = list(lens), page_size
        blocks = [-(-n // page_size) for n in lens]
        num_pages = sum(blocks) + 3
        self.pages = torch.randn((num_pages, 2, nkv, page_size, d), generator=gen, device=DEV).bfloat16()
        order = torch.randperm(num_pages, generator=gen, device=DEV).to(torch.int32)
        width = max(blocks)
        self.table = torch.full((len(lens), width), -1, dtype=torch.int32, device=DEV)
        at = 0
        for s, b in enumerate(blocks):
            self.table[s, :b] = order[at:at + b]
            at += b
        self.gen = gen

    def dense(self, s):
        b = -(-self.lens[s] // self.page_size)
        got = self.pages[self.table[s, :b].long()]                       # [b, 2, NKV, page, D]
        k = got[:, 0].permute(0, 2, 1, 3).reshape(-1, got.shape[2], got.shape[4])[:self.lens[s]]
        v = got[:, 1].permute(0, 2, 1, 3).reshape(-1, got.shape[2], got.shape[4])[:self.lens[s]]
        return k.float(), v.float()

    def plant(self, s, position, direction, strength):
        """Key `position` of sequence s (every kv head) points along `direction`."""
        page = int(self.table[s, position // self.page_size])
        self.pages[page, 0, :, position % self.page_size, :] = (direction * strength).bfloat16()


def launch(case, q_list, news, nh, nkv, d, window):
    """One step: sequence s brings news[s] queries (q_list[s]: [news[s], NH, D] bf16) at its last positions."""
    from microllm_rocm_b200.kernels import attention
    from microllm_rocm_b200.parts.base import StepContext
    pos0 = [l - n for l, n in zip(case.lens, news)]
    starts = [int(x) for x in np.cumsum([0] + list(news))]
    q = torch.cat([x.reshape(x.shape[0], nh * d) for x in q_list]).contiguous()
    positions = torch.cat([torch.arange(p, p + n, dtype=torch.int32) for p, n in zip(pos0, news)]).to(DEV)
    token_seq = torch.cat([torch.full((n,), s, dtype=torch.int32) for s, n in enumerate(news)]).to(DEV)
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = torch.full(q.shape, float("nan"), dtype=torch.bfloat16, device=DEV)
    ctx = StepContext(num_tokens=q.shape[0], num_seqs=len(news), token_ids=positions, positions=positions, token_seq=token_seq,
                      seq_starts=torch.tensor(starts, dtype=torch.int32, device=DEV),
                      seq_pos0=torch.tensor(pos0, dtype=torch.int32, device=DEV),
                      seq_lens=torch.tensor(case.lens, dtype=torch.int32, device=DEV), block_tables={}, state_slots=None,
                      logit_rows=None, error_flag=flag, seq_starts_host=starts, seq_pos0_host=pos0,
                      max_new_tokens=max(news), max_seq_len=max(case.lens))
    attention.paged_attention(q, case.pages, out, ctx, case.table, nh, nkv, d, 1.0 / math.sqrt(d), window)
    torch.cuda.synchronize()
    assert int(flag.item()) == 0
    plans = [v for k, v in ctx.extras.items() if isinstance(k, tuple) and k and k[0] == "attention_mma"]
    return out.float(), starts, pos0, plans


def worst_relative_error(got_rows, want_rows):
    """Largest |got - want| of a (row, head) over the largest |want| of that (row, head)."""
    err = (got_rows.double() - want_rows).abs().amax(dim=-1)
    size = want_rows.abs().amax(dim=-1).clamp_min(1e-3)
    return float((err / size).max())


PEAK = 3.0            # queries are scaled by this: a few dozen of thousands of keys carry the weight
PLANT = 16.0          # planted key and its queries: score 16 * 16 / sqrt(128) = 22.6 above everything else
BF16_ROW_TOL = 0.02   # of the row's largest value; measured worst 0.0066 (probabilities and outputs are rounded to bf16)


# ------------------------------------------------------------------------------ prompt portions (tcgen05 kernel)
@gpu
@pytest.mark.parametrize("context,new,window", [(2048, 2048, None), (2048, 2048, 1000), (8192, 8192, None), (8192, 8192, 1000),
                                                (6700, 700, None), (6700, 700, 3000)])
def test_long_prompt_portions_against_the_formula(context, new, window):
    """Whole prompts of 2,048 and 8,192 tokens and a portion that starts at position 6,000 (6 query heads per kv
    head, head size 128, 64-token pages): 128-row tiles that walk up to 64 key tiles, the ring of K/V stages
    wrapping many times, a window whose edge falls inside a key tile."""
    nh, nkv, d, page = 12, 2, 128, 64
    case = PagedCase([context], nkv, d, page, seed=context + new)
    gen = case.gen
    q = (torch.randn((new, nh, d), generator=gen, device=DEV) * PEAK).bfloat16()
    # heads 0..5 of every query row from the middle on point at a key in the first page (outside the window
    # when there is one: then it must NOT show)
    direction = torch.randn(d, generator=gen, device=DEV)
    direction /= direction.norm()
    far = 5
    case.plant(0, far, direction, PLANT)
    q[new // 2:, :6] = (direction * PLANT).bfloat16()
    out, starts, pos0, _ = launch(case, [q], [new], nh, nkv, d, window)
    out = out.reshape(new, nh, d)
    # rows: the edges of the 128-row tiles, of the window, and a few hundred random ones
    pick = {0, 1, 127, 128, 129, new // 2 - 1, new // 2, new - 129, new - 128, new - 1}
    if window is not None:
        pick |= {r for r in (window - 1 - pos0[0], window - pos0[0], far + window - 1 - pos0[0], far + window - pos0[0]) if 0 <= r < new}
    rng = np.random.default_rng(context)
    pick |= set(int(x) for x in rng.integers(0, new, 300))
    rows = torch.tensor(sorted(pick), device=DEV)
    k, v = case.dense(0)
    want = reference_rows(q[rows].float(), rows + pos0[0], k, v, window)
    assert torch.isfinite(out).all()
    worst = worst_relative_error(out[rows], want)
    print(f"long prompt {context}/{new} window {window}: worst relative row error {worst:.4f}")
    assert worst < BF16_ROW_TOL, worst
    # the planted key: seen by every later row without a window, by none whose window has passed it
    late = rows[rows >= new // 2]
    seen = (late + pos0[0] - far < window) if window is not None else torch.ones_like(late, dtype=torch.bool)
    target = v[far, 0]
    close = (out[late][:, 0] - target).abs().amax(dim=-1) < 0.05
    assert bool((close == seen).all())


# ------------------------------------------------------------------------------ decode steps (cluster kernel)
@gpu
@pytest.mark.parametrize("batch,context,nh,nkv,page,splits", [
    (1, 2073, 12, 2, 64, 16), (8, 2073, 12, 2, 64, 8), (64, 2073, 12, 2, 64, 2),
    (1, 8192, 12, 2, 64, 16), (8, 4096, 12, 2, 64, 8), (64, 4096, 12, 2, 64, 2), (8, 8192, 12, 2, 64, 8),
    (8, 8192, 40, 8, 64, 4), (2, 16500, 12, 2, 16, 8)])
@pytest.mark.parametrize("ring", [False, True])
def test_decode_steps_at_long_contexts_against_the_formula(batch, context, nh, nkv, page, splits, ring):
    """One decode step per case; the sequences of a batch differ in length (the longest has `context` tokens,
    the shortest a few hundred fewer, one of them only 40), so the CTAs of a cluster get uneven shares.  The last
    case has more than 1,024 blocks per sequence (16,500 tokens in 16-token pages): the block table no longer fits
    the kernel's shared-memory copy and is read from global memory.  Every case runs through both decode kernels:
    keys straight into registers, and keys through the ring of shared memory that TMA fills."""
    from microllm_rocm_b200.kernels import attention
    d = 128
    lens = [max(41, context - 37 * i) for i in range(batch)]
    if batch > 1:
        lens[-1] = 40
    case = PagedCase(lens, nkv, d, page, seed=batch * 100003 + context)
    gen = case.gen
    q = (torch.randn((batch, nh, d), generator=gen, device=DEV) * PEAK).bfloat16()
    direction = torch.randn(d, generator=gen, device=DEV)
    direction /= direction.norm()
    fars = []
    for s, n in enumerate(lens):                         # a planted key at a different place in every sequence
        far = (s * 997 + 3) % n
        fars.append(far)
        case.plant(s, far, direction, PLANT)
    q[:, :nh // 2] = (direction * PLANT).bfloat16()
    attention.DECODE_RING = ring
    try:
        out, _, _, plans = launch(case, [q[s:s + 1] for s in range(batch)], [1] * batch, nh, nkv, d, None)
    finally:
        attention.DECODE_RING = None
    assert plans and plans[0][3] == splits, f"planned clusters of {plans[0][3]}, the case is meant for {splits}"
    out = out.reshape(batch, nh, d)
    assert torch.isfinite(out).all()
    worst = 0.0
    for s, n in enumerate(lens):
        k, v = case.dense(s)
        want = reference_rows(q[s:s + 1].float(), torch.tensor([n - 1]), k, v, None)
        worst = max(worst, worst_relative_error(out[s:s + 1], want))
        group = nh // nkv
        for h in (0, nh // 2 - 1):
            assert (out[s, h] - v[fars[s], h // group]).abs().max() < 0.05, (s, h)
    print(f"decode batch {batch} context {context} heads {nh}/{nkv} clusters of {splits} ring {ring}: worst relative row error {worst:.4f}")
    assert worst < BF16_ROW_TOL, worst


@gpu
@pytest.mark.parametrize("ring", [False, True])
@pytest.mark.parametrize("nh,nkv", [(12, 2), (40, 8), (18, 1)])
def test_decoded_tokens_beside_a_prompt_portion_use_the_key_split(nh, nkv, ring):
    """A step that mixes a 300-token prompt portion with single tokens of sequences that already hold thousands of
    keys: the single tokens go through the decode shape (their keys split over a cluster), found through a list of
    their sequences, the portion through the tensor-memory kernel; each writes its own rows."""
    d, page = 128, 64
    lens = [3000, 2500, 41, 1717, 4000, 1]
    news = [1, 300, 1, 1, 1, 1]
    case = PagedCase(lens, nkv, d, page, seed=nh * 31 + nkv)
    gen = case.gen
    qs = [(torch.randn((n, nh, d), generator=gen, device=DEV) * PEAK).bfloat16() for n in news]
    direction = torch.randn(d, generator=gen, device=DEV)
    direction /= direction.norm()
    fars = [(s * 977 + 5) % n for s, n in enumerate(lens)]
    for s in (0, 3, 4):
        case.plant(s, fars[s], direction, PLANT)
        qs[s][:, :nh // 2] = (direction * PLANT).bfloat16()
    from microllm_rocm_b200.kernels import attention
    attention.DECODE_RING = ring
    try:
        out, starts, pos0, plans = launch(case, qs, news, nh, nkv, d, None)
    finally:
        attention.DECODE_RING = None
    assert plans and plans[0][7] == 5 * -(-(nh // nkv) // 16) and plans[0][8] > 1      # five listed sequences, keys split
    assert torch.isfinite(out).all()
    worst = 0.0
    for s, n in enumerate(lens):
        k, v = case.dense(s)
        rows = torch.arange(news[s], device=DEV)
        want = reference_rows(qs[s].float(), rows + pos0[s], k, v, None)
        got = out[starts[s]:starts[s + 1]].reshape(news[s], nh, d)
        worst = max(worst, worst_relative_error(got, want))
        if s in (0, 3, 4):
            assert (got[0, 0] - v[fars[s], 0]).abs().max() < 0.05, s
    print(f"decoded tokens beside a portion, heads {nh}/{nkv}: worst relative row error {worst:.4f}")
    assert worst < BF16_ROW_TOL, worst


# ------------------------------------------------------------------------------ two layers of the benchmark shape
@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_two_layers_of_the_benchmark_shape_against_the_plain_implementation(dtype, tmp_path_factory):
    """Two layers of the Qwen2.5-1.5B shape (width 1,536, 12/2 heads of 128, intermediate 8,960, vocabulary
    151,936, tied head) from a written model folder: a 2,048-token prompt in portions of 512, then 8 single
    tokens, 64-token pages.  Logits at the end of every portion and at every single token are held against the
    plain implementation, which runs the whole 2,056-token sequence on the CPU."""
    from microllm_rocm_b200.config import get_architecture, preset
    from microllm_rocm_b200.engine.loading import load_engine
    from microllm_rocm_b200.engine.step import StepEntry
    from microllm_rocm_b200.weights import write_random_model
    cfg = preset("qwen2.5-1.5b", num_hidden_layers=2)
    folder = str(tmp_path_factory.mktemp("two_layers_1p5b"))
    write_random_model(get_architecture("Qwen2ForCausalLM"), cfg, 5, folder, "bfloat16")
    gen = torch.Generator().manual_seed(11)
    tokens = torch.randint(0, cfg.vocab_size, (2056,), generator=gen).tolist()

    engine = load_engine(folder, dtype=dtype, page_size=64, max_tokens=2112, max_requests=2)
    engine.cache.add("r")
    rows, got = [], []
    for at in range(0, 2048, 512):
        got.append(engine.step([StepEntry("r", tokens[at:at + 512], [511])]))
        rows.append(at + 511)
    for at in range(2048, 2056):
        got.append(engine.step([StepEntry("r", tokens[at:at + 1], [0])]))
        rows.append(at)
    engine.check_device_errors()
    got = torch.cat([g.float().cpu() for g in got])
    del engine
    torch.cuda.empty_cache()

    # the plain implementation, part by part, with the head applied to the wanted rows only
    weights = plain.read_safetensors(os.path.join(folder, "model.safetensors"))
    raw = plain.read_config(os.path.join(folder, "config.json"))
    rnd = plain.Rounding(dtype)
    x = plain.embedding(weights["model.embed_tokens.weight"], tokens)
    for l in range(raw["num_hidden_layers"]):
        x = plain.block(x, weights, f"model.layers.{l}.", raw, list(range(len(tokens))), plain.layer_window(raw, l), rnd)
    x = rnd(plain.rms_norm(x[rows], weights["model.norm.weight"], raw["rms_norm_eps"]))
    want = plain.linear(x, weights["model.embed_tokens.weight"])

    assert torch.isfinite(got).all() and got.shape == want.shape
    err = (got - want).abs().amax(dim=1)
    size = want.abs().amax(dim=1)
    print(f"two layers of the 1.5B shape, {dtype}: worst |logit error| {float(err.max()):.3e} "
          f"at largest |logit| {float(size.max()):.3f}; per row relative {[round(float(e / s), 5) for e, s in zip(err, size)]}")
    limit = 3e-5 if dtype == "float32" else 0.02           # of the row's largest |logit|; measured 3.3e-6 and 0.0074
    assert bool((err <= limit * size).all()), (err / size).tolist()
