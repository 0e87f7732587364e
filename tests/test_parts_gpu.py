"""Each part alone, the run order as data, and a toy mixer with state of its own that a
test registers, builds and steps without touching the framework's files."""
import dataclasses
import json
import math
import os

import pytest
import torch

from tests.helpers import TINY, collect, make_folder, random_tokens, steps_mixed, steps_portions, steps_whole, tiny_config
from tests.plain import qwen2_plain as plain

pytestmark = pytest.mark.gpu
DEV = "cuda"


def runtime(dtype=torch.float32):
    from microllm_rocm_b200.parts import Runtime
    return Runtime(torch.device(DEV), dtype)


def simple_context(counts, pos0, page_size, tables=None, slots=None):
    """A StepContext for sequences that bring `counts[i]` tokens after `pos0[i]` cached ones."""
    import numpy as np
    from microllm_rocm_b200.parts.base import StepContext
    T, A = sum(counts), len(counts)
    starts = [0]
    for c in counts:
        starts.append(starts[-1] + c)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    positions = [p + i for p, c in zip(pos0, counts) for i in range(c)]
    seq = [a for a, c in enumerate(counts) for _ in range(c)]
    return StepContext(num_tokens=T, num_seqs=A, token_ids=i32([0] * T), positions=i32(positions), token_seq=i32(seq),
                       seq_starts=i32(starts), seq_pos0=i32(pos0), seq_lens=i32([p + c for p, c in zip(pos0, counts)]),
                       block_tables=tables or {}, state_slots=i32(slots or list(range(A))), logit_rows=i32([T - 1]),
                       error_flag=torch.zeros(1, dtype=torch.int32, device=DEV), seq_starts_host=starts,
                       seq_pos0_host=list(pos0), state_slots_host=slots or list(range(A)), max_new_tokens=max(counts),
                       max_seq_len=max(p + c for p, c in zip(pos0, counts)))


def test_norm_part_alone():
    from microllm_rocm_b200.parts.norm import RMSNorm
    n = RMSNorm(dict(size=100, eps=1e-5), runtime())
    assert n.weight_specs()["weight"].shape == (100,)
    w = 1 + 0.1 * torch.randn(100)
    n.bind({"weight": w.to(DEV)})
    x = torch.randn(7, 100)
    out = torch.empty(7, 100, device=DEV)
    n.forward(x.to(DEV), out)
    assert torch.allclose(out.cpu(), plain.rms_norm(x, w, 1e-5), atol=2e-5)


def test_rotary_part_tables():
    from microllm_rocm_b200.parts.rotary import RotaryEmbedding
    r = RotaryEmbedding(dict(head_dim=32, theta=1e6), runtime())
    t = r.rotary_table(32)
    assert t.rotary_dim == 32 and not t.interleaved and t.inv_freq.shape == (16,)
    assert abs(float(t.inv_freq[1]) - 1e6 ** (-2 / 32)) < 1e-7
    half = RotaryEmbedding(dict(head_dim=32, rotary_dim=16, theta=1e4, layout="interleaved"), runtime()).rotary_table(32)
    assert half.rotary_dim == 16 and half.interleaved and half.inv_freq.shape == (8,)
    with pytest.raises(ValueError):
        RotaryEmbedding(dict(head_dim=32, rotary_dim=34, theta=1e4), runtime())


def test_feed_forward_part_alone():
    from microllm_rocm_b200.parts.mlp import SwiGLU
    ff = SwiGLU(dict(hidden_size=48, intermediate_size=100), runtime())
    g, u, d = torch.randn(100, 48) * 0.2, torch.randn(100, 48) * 0.2, torch.randn(48, 100) * 0.2
    ff.bind({"gate_proj.weight": g.to(DEV), "up_proj.weight": u.to(DEV), "down_proj.weight": d.to(DEV)})
    x = torch.randn(5, 48)
    got = ff.forward(x.to(DEV), None).cpu()
    want = plain.linear(plain.swiglu(plain.linear(x, g), plain.linear(x, u)), d)
    assert torch.allclose(got, want, atol=2e-5)


@pytest.mark.parametrize("window", [None, 6])
def test_attention_part_alone_over_two_steps(window):
    """The mixer with its cache view: a prompt in one step, then two more tokens, against the
    plain attention over the whole sequence."""
    from microllm_rocm_b200.parts.attention import Attention
    from microllm_rocm_b200.parts.base import PagedKVView
    from microllm_rocm_b200.parts.rotary import RotaryEmbedding
    torch.manual_seed(0)
    H, NH, NKV, D, T = 40, 6, 3, 16, 13
    rt = runtime()
    rot = RotaryEmbedding(dict(head_dim=D, theta=1e4), rt)
    att = Attention(dict(hidden_size=H, num_heads=NH, num_kv_heads=NKV, head_dim=D, qkv_bias=True, window=window), rt, rot)
    need = att.cache_need()
    assert (need.num_kv_heads, need.head_dim, need.window) == (NKV, D, window)
    w = {n: torch.randn(s.shape) * 0.2 for n, s in att.weight_specs().items()}
    att.bind({n: t.to(DEV) for n, t in w.items()})
    x = torch.randn(T, H)
    # plain
    q = plain.linear(x, w["q_proj.weight"], w["q_proj.bias"]).view(T, NH, D)
    k = plain.linear(x, w["k_proj.weight"], w["k_proj.bias"]).view(T, NKV, D)
    v = plain.linear(x, w["v_proj.weight"], w["v_proj.bias"]).view(T, NKV, D)
    q, k = plain.rope_split_half(q, range(T), 1e4), plain.rope_split_half(k, range(T), 1e4)
    want = plain.linear(plain.causal_gqa_attention(q, k, v, window).reshape(T, NH * D), w["o_proj.weight"])
    # engine part: pages 3, 0, 2 hold blocks 0, 1, 2
    pages = torch.zeros(4, 2, NKV, 8, D, device=DEV)
    table = torch.tensor([[3, 0, 2]], dtype=torch.int32, device=DEV)
    view = PagedKVView(pages, table, 8, True)
    got = []
    for begin, end in ((0, 11), (11, 12), (12, 13)):
        ctx = simple_context([end - begin], [begin], 8)
        got.append(att.forward(x[begin:end].to(DEV), ctx, view).cpu())
        assert int(ctx.error_flag.item()) == 0
    assert torch.allclose(torch.cat(got), want, atol=2e-5)
    assert pages[1].abs().sum() == 0, "page 1 is not in the table and must stay untouched"


# --------------------------------------------------------------------------------- order as data
def plain_block_with_shared_kv(x, w, prefix, cfg, positions, window, shared=None):
    """tests/plain block, returning its rotated k and v, or using `shared` ones instead."""
    H, NH, NKV = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"]
    D, eps, T = H // NH, cfg["rms_norm_eps"], x.shape[0]
    h = plain.rms_norm(x, w[prefix + "input_layernorm.weight"], eps)
    a = prefix + "self_attn."
    q = plain.rope_split_half(plain.linear(h, w[a + "q_proj.weight"], w[a + "q_proj.bias"]).view(T, NH, D), positions, cfg["rope_theta"])
    if shared is None:
        k = plain.rope_split_half(plain.linear(h, w[a + "k_proj.weight"], w[a + "k_proj.bias"]).view(T, NKV, D), positions, cfg["rope_theta"])
        v = plain.linear(h, w[a + "v_proj.weight"], w[a + "v_proj.bias"]).view(T, NKV, D)
    else:
        k, v = shared
    x = x + plain.linear(plain.causal_gqa_attention(q, k, v, window).reshape(T, NH * D), w[a + "o_proj.weight"])
    h = plain.rms_norm(x, w[prefix + "post_attention_layernorm.weight"], eps)
    m = prefix + "mlp."
    x = x + plain.linear(plain.swiglu(plain.linear(h, w[m + "gate_proj.weight"]), plain.linear(h, w[m + "up_proj.weight"])), w[m + "down_proj.weight"])
    return x, (k, v)


def test_a_layer_may_run_twice_and_a_run_may_read_another_runs_cache(tmp_path_factory):
    """order = [L0, L1, L0 again (cache of its own), L1 reading the cache of the first L1 run]."""
    from microllm_rocm_b200.config import get_architecture
    from microllm_rocm_b200.config.spec import RunSpec
    from microllm_rocm_b200.engine.loading import make_engine
    from microllm_rocm_b200.parts import build_model
    from microllm_rocm_b200.weights import load_weights
    folder = make_folder(tmp_path_factory, "a")
    cfg = tiny_config("a")
    spec = get_architecture("Qwen2ForCausalLM").build_spec(cfg)
    spec = dataclasses.replace(spec, order=[RunSpec(0), RunSpec(1), RunSpec(0), RunSpec(1, read_cache_of=1)])
    model = build_model(spec, runtime())
    assert sorted(model.cache_entries) == ["run0", "run1", "run2"]
    load_weights(model, folder)
    engine = make_engine(model, 16, 32, 4)
    toks = random_tokens(45, cfg.vocab_size, 9)
    reqs = {"x": toks}
    whole = collect(engine, steps_whole(reqs))
    cut = collect(engine, steps_portions(reqs))
    w = plain.read_safetensors(os.path.join(folder, "model.safetensors"))
    raw = plain.read_config(os.path.join(folder, "config.json"))
    pos = list(range(len(toks)))
    x = plain.embedding(w["model.embed_tokens.weight"], toks)
    x, _ = plain_block_with_shared_kv(x, w, "model.layers.0.", raw, pos, None)
    x, kv1 = plain_block_with_shared_kv(x, w, "model.layers.1.", raw, pos, None)
    x, _ = plain_block_with_shared_kv(x, w, "model.layers.0.", raw, pos, None)
    x, _ = plain_block_with_shared_kv(x, w, "model.layers.1.", raw, pos, None, shared=kv1)
    want = plain.linear(plain.rms_norm(x, w["model.norm.weight"], raw["rms_norm_eps"]), w["model.embed_tokens.weight"])
    for p in pos:
        assert torch.allclose(whole[("x", p)], want[p], atol=2e-5), p
        assert torch.equal(whole[("x", p)], cut[("x", p)])


# --------------------------------------------------------------------------------- a toy mixer with state
def register_toy():
    """A mixer whose output at a token is W applied to the running mean of all inputs of its
    sequence so far: it needs fixed-size state per request (a sum and a count), carried
    across steps, and no pages.  Defined here; the framework's files know nothing of it."""
    from microllm_rocm_b200.config import Architecture, register_architecture
    from microllm_rocm_b200.config.spec import LayerSpec, ModelSpec, PartSpec, RunSpec
    from microllm_rocm_b200.parts import FixedStateNeed, Mixer, WeightSpec, register_mixer

    @register_mixer("toy_running_mean", replace=True)
    class RunningMean(Mixer):
        def __init__(self, params, rt, position=None):
            self.prefix, self.h, self.rt = params.get("prefix", ""), int(params["hidden_size"]), rt

        def cache_need(self):
            return FixedStateNeed((self.h + 1,), torch.float32)

        def weight_specs(self):
            return {"mix.weight": WeightSpec((self.h, self.h))}

        def bind(self, tensors):
            self.w = tensors["mix.weight"]

        def forward(self, x, ctx, cache):
            out = torch.empty(x.shape, dtype=torch.float32, device=x.device)
            for a in range(ctx.num_seqs):
                lo, hi = ctx.seq_starts_host[a], ctx.seq_starts_host[a + 1]
                state = cache.storage[cache.slots_host[a]]
                if ctx.seq_pos0_host[a] == 0:
                    state.zero_()                               # a slot that is used again starts clean
                sums = state[:self.h] + torch.cumsum(x[lo:hi].float(), 0)
                counts = state[self.h] + torch.arange(1, hi - lo + 1, device=x.device, dtype=torch.float32)
                out[lo:hi] = (sums / counts[:, None]) @ self.w.float().t()
                if cache.writable:
                    state[:self.h] = sums[-1]
                    state[self.h] = counts[-1]
            return out

    @register_mixer("toy_planned_scale", replace=True)
    class PlannedScale(Mixer):
        """W x scaled by a factor that depends on the token's position, looked up in a device table that the mixer
        PLANS on the host for the longest sequence of the step and keeps in ctx.extras.  A captured decode step
        freezes the table it was captured with: beyond the table's end the lookup is clamped and the result
        wrong, unless whoever holds the context asks plan_stale() and lets the mixer plan anew."""
        graph_safe = True                 # device-resident inputs only: positions and the planned table
        PLAN_KEY = ("toy_planned_scale", "table")
        GRANULE = 16
        plans_made = 0

        def __init__(self, params, rt, position=None):
            self.prefix, self.h, self.rt = params.get("prefix", ""), int(params["hidden_size"]), rt

        def weight_specs(self):
            return {"mix.weight": WeightSpec((self.h, self.h))}

        def bind(self, tensors):
            self.w = tensors["mix.weight"]

        @classmethod
        def capacity_for(cls, max_seq_len):
            return -(-max(1, max_seq_len) // cls.GRANULE) * cls.GRANULE

        def plan_group(self):
            return self.PLAN_KEY

        def plan_stale(self, ctx, max_seq_len):
            table = ctx.extras.get(self.PLAN_KEY)
            return table is not None and table.shape[0] != self.capacity_for(max_seq_len)

        def forget_plans(self, ctx):
            ctx.extras.pop(self.PLAN_KEY, None)

        def forward(self, x, ctx, cache):
            table = ctx.extras.get(self.PLAN_KEY)
            if table is None or (not ctx.decode_only and table.shape[0] < self.capacity_for(ctx.max_seq_len)):
                capacity = self.capacity_for(ctx.max_seq_len)
                table = ctx.extras[self.PLAN_KEY] = 1.0 + 0.25 * (torch.arange(capacity, device=x.device) // 8).float()
                type(self).plans_made += 1
            scale = table[torch.clamp(ctx.positions.long(), max=table.shape[0] - 1)]
            return (x.float() @ self.w.float().t()) * scale[:, None]

    @dataclasses.dataclass(frozen=True)
    class ToyConfig:
        vocab_size: int
        hidden_size: int
        intermediate_size: int
        kinds: tuple                      # per layer: "attention" or "toy"
        num_heads: int = 2
        eps: float = 1e-5
        max_position_embeddings: int = 256
        torch_dtype: str = "float32"

        @classmethod
        def from_dict(cls, raw):
            return cls(raw["vocab_size"], raw["hidden_size"], raw["intermediate_size"], tuple(raw["kinds"]),
                       raw.get("num_heads", 2), raw.get("eps", 1e-5), raw.get("max_position_embeddings", 256))

        def to_dict(self):
            d = dataclasses.asdict(self)
            d["kinds"] = list(self.kinds)
            d["architectures"] = ["ToyForCausalLM"]
            return d

    def build_spec(cfg):
        h = cfg.hidden_size
        norm = lambda sub: PartSpec("rmsnorm", dict(prefix=sub, size=h, eps=cfg.eps))
        layers = []
        for l, kind in enumerate(cfg.kinds):
            mixer = (PartSpec("attention", dict(prefix="attn.", hidden_size=h, num_heads=cfg.num_heads, num_kv_heads=1,
                                                head_dim=h // cfg.num_heads, qkv_bias=False, window=None))
                     if kind == "attention" else
                     PartSpec("toy_planned_scale", dict(prefix="toy.", hidden_size=h)) if kind == "planned" else
                     PartSpec("toy_running_mean", dict(prefix="toy.", hidden_size=h)))
            layers.append(LayerSpec(prefix=f"layers.{l}.", block=PartSpec("pre_norm_residual"), mixer_norm=norm("n1."),
                                    mixer=mixer, ffn_norm=norm("n2."),
                                    feed_forward=PartSpec("swiglu", dict(prefix="ff.", hidden_size=h,
                                                                         intermediate_size=cfg.intermediate_size))))
        return ModelSpec(architecture="ToyForCausalLM", hidden_size=h, vocab_size=cfg.vocab_size,
                         max_position=cfg.max_position_embeddings,
                         embedding=PartSpec("token_embedding", dict(name="embed.weight", vocab_size=cfg.vocab_size, hidden_size=h)),
                         position=PartSpec("rotary", dict(head_dim=h // cfg.num_heads, theta=10000.0)),
                         layers=layers, order=[RunSpec(l) for l in range(len(layers))], final_norm=norm("final."),
                         head=PartSpec("lm_head", dict(name="head.weight", vocab_size=cfg.vocab_size, hidden_size=h, tied_to=None)))

    arch = Architecture("ToyForCausalLM", ToyConfig, build_spec)
    register_architecture(arch, replace=True)
    return arch, ToyConfig


def plain_toy_forward(w, cfg, toks):
    T, H, NH = len(toks), cfg.hidden_size, cfg.num_heads
    D = H // NH
    pos = list(range(T))
    x = plain.embedding(w["embed.weight"], toks)
    for l, kind in enumerate(cfg.kinds):
        p = f"layers.{l}."
        h = plain.rms_norm(x, w[p + "n1.weight"], cfg.eps)
        if kind == "attention":
            q = plain.rope_split_half(plain.linear(h, w[p + "attn.q_proj.weight"]).view(T, NH, D), pos, 10000.0)
            k = plain.rope_split_half(plain.linear(h, w[p + "attn.k_proj.weight"]).view(T, 1, D), pos, 10000.0)
            v = plain.linear(h, w[p + "attn.v_proj.weight"]).view(T, 1, D)
            x = x + plain.linear(plain.causal_gqa_attention(q, k, v, None).reshape(T, H), w[p + "attn.o_proj.weight"])
        elif kind == "planned":
            scale = 1.0 + 0.25 * (torch.arange(T) // 8).float()
            x = x + plain.linear(h, w[p + "toy.mix.weight"]) * scale[:, None]
        else:
            mean = torch.cumsum(h, 0) / torch.arange(1, T + 1, dtype=torch.float32)[:, None]
            x = x + plain.linear(mean, w[p + "toy.mix.weight"])
        h = plain.rms_norm(x, w[p + "n2.weight"], cfg.eps)
        x = x + plain.linear(plain.swiglu(plain.linear(h, w[p + "ff.gate_proj.weight"]), plain.linear(h, w[p + "ff.up_proj.weight"])),
                             w[p + "ff.down_proj.weight"])
    return plain.linear(plain.rms_norm(x, w["final.weight"], cfg.eps), w["head.weight"])


def test_a_toy_mixer_with_state_is_registered_built_and_stepped(tmp_path):
    from microllm_rocm_b200.engine.loading import load_engine
    from microllm_rocm_b200.weights import write_random_model
    arch, ToyConfig = register_toy()
    cfg = ToyConfig(vocab_size=90, hidden_size=32, intermediate_size=56, kinds=("toy", "attention", "toy"))
    folder = write_random_model(arch, cfg, 4, str(tmp_path / "toy"), "float32")
    assert json.load(open(os.path.join(folder, "config.json")))["architectures"] == ["ToyForCausalLM"]
    engine = load_engine(folder, dtype="float32", page_size=16, max_tokens=256, max_requests=3)
    # one paged entry (the attention layer), two state entries (the toy layers)
    assert sorted(engine.cache.entry_group) == ["run1"] and sorted(engine.cache.state_storage) == ["run0", "run2"]
    reqs = {f"q{i}": random_tokens(n, cfg.vocab_size, n) for i, n in enumerate([40, 23, 57, 31, 18])}
    w = plain.read_safetensors(os.path.join(folder, "model.safetensors"))
    whole = collect(engine, steps_whole(reqs))
    for rid, toks in reqs.items():
        want = plain_toy_forward(w, cfg, toks)
        for p in range(len(toks)):
            assert torch.allclose(whole[(rid, p)], want[p], atol=3e-5), (rid, p)
    # state carried across portions, and slots used again by later requests, give the same logits
    steps, peak = steps_mixed(reqs, max_live=3, seed=2)
    mixed = collect(load_engine(folder, dtype="float32", page_size=16, max_tokens=peak, max_requests=3), steps)
    for key, row in whole.items():
        assert torch.allclose(mixed[key], row, atol=3e-5), key


def test_a_toy_mixer_freezes_a_plan_into_a_captured_decode_step_and_plans_anew(tmp_path):
    """A mixer defined here keeps a host-made launch plan (a table sized for the longest sequence) in the step
    context; steady decoding captures the step, plan included.  The engine asks the mixer's own hooks whether the
    plan still suits the context and lets it plan anew: generation through captured steps equals generation
    step by step and the plain forward, across three sizes of the table.  Nothing under the package names this mixer."""
    from microllm_rocm_b200.engine.llm import LLM
    from microllm_rocm_b200.parts.base import MIXERS
    from microllm_rocm_b200.sampling import GenerationConfig
    from microllm_rocm_b200.weights import write_random_model
    arch, ToyConfig = register_toy()
    cfg = ToyConfig(vocab_size=90, hidden_size=32, intermediate_size=56, kinds=("planned", "attention", "planned"))
    folder = write_random_model(arch, cfg, 6, str(tmp_path / "planned"), "float32")
    planned = MIXERS["toy_planned_scale"]
    prompt = random_tokens(10, cfg.vocab_size, 3)
    greedy = GenerationConfig(max_new_tokens=30, temperature=0.0)

    stepwise = LLM(folder, dtype="float32", max_tokens=256, max_seqs=2, cuda_graphs=False)
    want = stepwise.generate([prompt], greedy)[0]

    llm = LLM(folder, dtype="float32", max_tokens=256, max_seqs=2, cuda_graphs=True)
    assert llm.graphs is not None, "the toy mixer says it is graph safe"
    planned.plans_made = 0
    got = llm.generate([prompt], greedy)[0]
    assert got == want
    # lengths 11..40 pass the table sizes 16, 32 and 48: planned for the prompt, then once per size
    assert planned.plans_made >= 3 and llm.graphs.captures >= 3, (planned.plans_made, llm.graphs.captures)
    assert llm.graph_steps >= 25

    w = plain.read_safetensors(os.path.join(folder, "model.safetensors"))
    logits = plain_toy_forward(w, cfg, prompt + got)
    for i, token in enumerate(got):
        row = logits[len(prompt) + i - 1]
        assert int(row.argmax()) == token or float(row.max() - row[token]) < 1e-4, i


# --------------------------------------------------------------------------------- more toy parts: routing, positions, a norm
def register_toy_routed():
    """Three more kinds defined in the test: a feed-forward that ROUTES every token to one of E small experts
    (top-1 of a linear router, fp32 softmax weight on the chosen expert), a position encoding that ADDS a
    learned vector per absolute position to the embedded tokens (and gives the attention nothing to rotate),
    and a norm that subtracts the mean (LayerNorm with weight and bias).  The framework's files know none
    of them; they meet the framework's attention, block, embedding and head in one model."""
    from microllm_rocm_b200.config import Architecture, register_architecture
    from microllm_rocm_b200.config.spec import LayerSpec, ModelSpec, PartSpec, RunSpec
    from microllm_rocm_b200.parts import (FeedForward, Norm, PositionEncoding, WeightSpec, register_feed_forward,
                                          register_norm, register_position_encoding)

    @register_feed_forward("toy_routed", replace=True)
    class Routed(FeedForward):
        def __init__(self, params, rt):
            self.prefix, self.rt = params.get("prefix", ""), rt
            self.h, self.i, self.e = int(params["hidden_size"]), int(params["intermediate_size"]), int(params["experts"])

        def weight_specs(self):
            specs = {"router.weight": WeightSpec((self.e, self.h), init=("normal", 0.5))}
            for e in range(self.e):
                specs[f"experts.{e}.up.weight"] = WeightSpec((self.i, self.h), init=("normal", 0.2))
                specs[f"experts.{e}.down.weight"] = WeightSpec((self.h, self.i), init=("normal", 0.2))
            return specs

        def bind(self, tensors):
            self.router = tensors["router.weight"]
            self.up = [tensors[f"experts.{e}.up.weight"] for e in range(self.e)]
            self.down = [tensors[f"experts.{e}.down.weight"] for e in range(self.e)]

        def forward(self, x, ctx):
            x = x.float()
            weights = torch.softmax(x @ self.router.float().t(), dim=-1)           # router logits and softmax in fp32
            chosen = weights.argmax(-1)
            out = torch.zeros_like(x)
            for e in range(self.e):
                rows = (chosen == e).nonzero().flatten()
                if rows.numel():
                    hidden = torch.relu(x[rows] @ self.up[e].float().t())
                    out[rows] = weights[rows, e, None] * (hidden @ self.down[e].float().t())
            return out

    @register_position_encoding("toy_learned", replace=True)
    class Learned(PositionEncoding):
        def __init__(self, params, rt):
            self.prefix, self.n, self.h = params.get("prefix", ""), int(params["positions"]), int(params["hidden_size"])

        def weight_specs(self):
            return {"table.weight": WeightSpec((self.n, self.h), init=("normal", 0.3))}

        def bind(self, tensors):
            self.table = tensors["table.weight"]

        def on_embedding(self, x, ctx):
            x += self.table.float()[ctx.positions.long()]

    @register_norm("toy_layernorm", replace=True)
    class LayerNorm(Norm):
        def __init__(self, params, rt):
            self.prefix, self.size, self.eps = params.get("prefix", ""), int(params["size"]), float(params["eps"])

        def weight_specs(self):
            return {"weight": WeightSpec((self.size,), role="vector", init=("one_plus_normal", 0.1)),
                    "bias": WeightSpec((self.size,), role="vector", init=("normal", 0.1))}

        def bind(self, tensors):
            self.weight, self.bias = tensors["weight"], tensors["bias"]

        def forward(self, x, out, rows=None):
            x = x if rows is None else x[rows.long()]
            out.copy_(torch.nn.functional.layer_norm(x.float(), (self.size,), self.weight, self.bias, self.eps))

        def add_forward(self, residual, delta, out):
            residual += delta if delta.dim() == 2 else delta.sum(0)       # a delta may be partial sums [S, T, H]
            self.forward(residual, out)

    @dataclasses.dataclass(frozen=True)
    class RoutedConfig:
        vocab_size: int
        hidden_size: int
        intermediate_size: int
        experts: int
        layers: int
        num_heads: int = 2
        eps: float = 1e-5
        max_position_embeddings: int = 128
        torch_dtype: str = "float32"

        @classmethod
        def from_dict(cls, raw):
            return cls(raw["vocab_size"], raw["hidden_size"], raw["intermediate_size"], raw["experts"], raw["layers"],
                       raw.get("num_heads", 2), raw.get("eps", 1e-5), raw.get("max_position_embeddings", 128))

        def to_dict(self):
            return dict(dataclasses.asdict(self), architectures=["ToyRoutedForCausalLM"])

    def build_spec(cfg):
        h = cfg.hidden_size
        norm = lambda sub: PartSpec("toy_layernorm", dict(prefix=sub, size=h, eps=cfg.eps))
        layers = [LayerSpec(prefix=f"layers.{l}.", block=PartSpec("pre_norm_residual"), mixer_norm=norm("n1."),
                            mixer=PartSpec("attention", dict(prefix="attn.", hidden_size=h, num_heads=cfg.num_heads, num_kv_heads=1,
                                                             head_dim=h // cfg.num_heads, qkv_bias=True, window=None)),
                            ffn_norm=norm("n2."),
                            feed_forward=PartSpec("toy_routed", dict(prefix="ff.", hidden_size=h, experts=cfg.experts,
                                                                     intermediate_size=cfg.intermediate_size)))
                  for l in range(cfg.layers)]
        return ModelSpec(architecture="ToyRoutedForCausalLM", hidden_size=h, vocab_size=cfg.vocab_size,
                         max_position=cfg.max_position_embeddings,
                         embedding=PartSpec("token_embedding", dict(name="embed.weight", vocab_size=cfg.vocab_size, hidden_size=h)),
                         position=PartSpec("toy_learned", dict(prefix="positions.", positions=cfg.max_position_embeddings, hidden_size=h)),
                         layers=layers, order=[RunSpec(l) for l in range(len(layers))], final_norm=norm("final."),
                         head=PartSpec("lm_head", dict(name="head.weight", vocab_size=cfg.vocab_size, hidden_size=h, tied_to=None)))

    arch = Architecture("ToyRoutedForCausalLM", RoutedConfig, build_spec)
    register_architecture(arch, replace=True)
    return arch, RoutedConfig


def plain_routed_forward(w, cfg, toks):
    T, H, NH = len(toks), cfg.hidden_size, cfg.num_heads
    D = H // NH
    ln = lambda x, p: torch.nn.functional.layer_norm(x, (H,), w[p + "weight"], w[p + "bias"], cfg.eps)
    x = plain.embedding(w["embed.weight"], toks) + w["positions.table.weight"][:T]
    for l in range(cfg.layers):
        p = f"layers.{l}."
        h = ln(x, p + "n1.")
        q = (plain.linear(h, w[p + "attn.q_proj.weight"]) + w[p + "attn.q_proj.bias"]).view(T, NH, D)
        k = (plain.linear(h, w[p + "attn.k_proj.weight"]) + w[p + "attn.k_proj.bias"]).view(T, 1, D)
        v = (plain.linear(h, w[p + "attn.v_proj.weight"]) + w[p + "attn.v_proj.bias"]).view(T, 1, D)
        x = x + plain.linear(plain.causal_gqa_attention(q, k, v, None).reshape(T, H), w[p + "attn.o_proj.weight"])
        h = ln(x, p + "n2.")
        weights = torch.softmax(plain.linear(h, w[p + "ff.router.weight"]), -1)
        out = torch.zeros_like(h)
        for t in range(T):
            e = int(weights[t].argmax())
            hidden = torch.relu(plain.linear(h[t:t + 1], w[p + f"ff.experts.{e}.up.weight"]))
            out[t] = weights[t, e] * plain.linear(hidden, w[p + f"ff.experts.{e}.down.weight"])[0]
        x = x + out
    return plain.linear(ln(x, "final."), w["head.weight"])


def test_toy_routing_positions_and_norm_are_registered_built_and_stepped(tmp_path):
    """A routed feed-forward, learned positions and a layer norm, all defined in this file, build into a model
    beside the framework's attention (which then rotates nothing), load from a folder written by the
    random-weights mode, and step whole and in mixed portions to the same logits as a plain forward."""
    from microllm_rocm_b200.engine.loading import load_engine
    from microllm_rocm_b200.weights import write_random_model
    arch, RoutedConfig = register_toy_routed()
    cfg = RoutedConfig(vocab_size=70, hidden_size=48, intermediate_size=40, experts=3, layers=2, num_heads=3)
    folder = write_random_model(arch, cfg, 7, str(tmp_path / "routed"), "float32")
    engine = load_engine(folder, dtype="float32", page_size=16, max_tokens=256, max_requests=3)
    reqs = {f"q{i}": random_tokens(n, cfg.vocab_size, 3 * n) for i, n in enumerate([33, 50, 12, 41])}
    w = plain.read_safetensors(os.path.join(folder, "model.safetensors"))
    whole = collect(engine, steps_whole(reqs))
    experts_used = set()
    for rid, toks in reqs.items():
        want = plain_routed_forward(w, cfg, toks)
        for p in range(len(toks)):
            assert torch.allclose(whole[(rid, p)], want[p], atol=5e-5), (rid, p)
        h0 = torch.nn.functional.layer_norm(plain.embedding(w["embed.weight"], toks) + w["positions.table.weight"][:len(toks)],
                                            (cfg.hidden_size,), w["layers.0.n1.weight"], w["layers.0.n1.bias"], cfg.eps)
        experts_used |= set(plain.linear(h0, w["layers.0.ff.router.weight"]).argmax(-1).tolist())
    assert len(experts_used) > 1                      # the router really sends tokens to different experts
    steps, peak = steps_mixed(reqs, max_live=3, seed=4)
    mixed = collect(load_engine(folder, dtype="float32", page_size=16, max_tokens=peak, max_requests=3), steps)
    for key, row in whole.items():
        assert torch.allclose(mixed[key], row, atol=5e-5), key
