"""Generality of the parts: toy parts and a toy architecture, defined here in the test, are
registered, built, loaded from a model folder made by the random-weights mode and stepped
through the framework's step function, without any change to the framework's files.

The toys: a mixer with state of its own (a per-channel running average kept in the request's
state slot), a position encoding that rotates neighbouring pairs, a feed-forward with routing
(top-1 of two small experts), and an order of layers that names one block twice and lets a
layer read another layer's cache.  They stand for no model of anyone's."""
from dataclasses import asdict, dataclass

import pytest
import torch

import plain_qwen3 as plain
from part_helpers import tolerance

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]


def define_toys():
    import kirai_b200
    from kirai_b200.models.plan import LayerCall, ModelPlan
    from kirai_b200.parts import Block, Embedding, GQAttention, Linear, OutputHead, RMSNorm, SwiGLU
    from kirai_b200.parts.base import FeedForward, Mixer, PositionEncoding, StateNeed, WeightSpec

    class RunningAverageMixer(Mixer):
        """state <- decay * state + x_t ; out_t = state * gain   (state [H] per request, in its slot)."""

        def __init__(self, name, width, decay):
            self.name, self.width, self.decay = name, width, decay

        def cache_need(self):
            return StateNeed((self.width,), torch.float32)

        def weight_specs(self):
            return {self.name: WeightSpec((self.width,), "norm")}

        def load(self, weights, rt):
            self.rt = rt
            self.gain = weights.on_device(self.name, torch.float32)

        def forward(self, x, batch, cache, write_cache=True):
            out = torch.empty_like(x)
            for r in range(batch.num_requests):
                first = sum(batch.query_lens[:r])
                state = cache.state[batch.slot_ids[r]]
                for t in range(first, first + batch.query_lens[r]):  # a request's tokens in order
                    state.mul_(self.decay).add_(x[t].float())
                    out[t] = (state * self.gain).to(x.dtype)
            return out

    class DeviceRunningAverageMixer(RunningAverageMixer):
        """The same mixer, fit for a captured decode step: when every request brings one token it reads the
        requests' slots on the device and advances each state once, with no host loop."""

        capture_safe = True

        def forward(self, x, batch, cache, write_cache=True):
            if batch.max_query_len != 1:
                return super().forward(x, batch, cache, write_cache)
            slots = batch.slots.long()
            state = cache.state.index_select(0, slots) * self.decay + x.float()
            cache.state.index_copy_(0, slots, state)
            return (state * self.gain).to(x.dtype)

    class NeighbourPairRotation(PositionEncoding):
        """Rotates the pairs (2i, 2i + 1) by position * theta^(-i / (d/2)): another pairing than the half split."""

        def __init__(self, head_dim, theta, capture_safe=False):
            self.head_dim, self.theta, self.capture_safe = head_dim, theta, capture_safe  # device arithmetic only

        def load(self, weights, rt):
            self.rt = rt
            half = self.head_dim // 2
            self.freq = torch.pow(torch.tensor(self.theta), -torch.arange(half, dtype=torch.float32) / half).to(rt.device)

        def apply(self, q, k, positions):
            angle = positions.float()[:, None, None] * self.freq[None, None, :]
            cos, sin = torch.cos(angle), torch.sin(angle)
            for x in (q, k):
                even, odd = x[..., 0::2].float(), x[..., 1::2].float()  # views of x when x is 32-bit
                new_even, new_odd = even * cos - odd * sin, odd * cos + even * sin
                x[..., 0::2] = new_even.to(x.dtype)
                x[..., 1::2] = new_odd.to(x.dtype)

    class TopOneOfTwo(FeedForward):
        """A router picks one of two SwiGLU experts per token (router logits in 32-bit)."""

        def __init__(self, prefix, hidden, inter, on_device=False):
            self.router = Linear([(prefix + "router.weight", 2)], hidden)
            self.experts = [SwiGLU(prefix + f"experts.{e}.", hidden, inter) for e in range(2)]
            # gathering each expert's rows needs their count on the host; the device form runs both experts on every
            # row and keeps the chosen one, which a captured step can do
            self.capture_safe = self.on_device = on_device

        def weight_specs(self):
            specs = dict(self.router.weight_specs())
            for expert in self.experts:
                specs.update(expert.weight_specs())
            return specs

        def load(self, weights, rt):
            self.rt = rt
            self.router.load(weights, rt)
            for expert in self.experts:
                expert.load(weights, rt)

        def forward(self, x, batch=None):
            choice = self.router.forward(x, torch.float32).argmax(dim=-1)
            if self.on_device:
                both = [expert.forward(x) for expert in self.experts]
                return torch.where((choice == 0)[:, None], both[0], both[1])
            out = torch.zeros_like(x)
            for e, expert in enumerate(self.experts):
                rows = (choice == e).nonzero().flatten()
                if rows.numel():
                    out[rows] = expert.forward(x[rows].contiguous())
            return out

    @dataclass(frozen=True)
    class ToyConfig:
        hidden_size: int = 48
        vocab_size: int = 200
        head_dim: int = 16
        heads: int = 3
        kv_heads: int = 1
        inter: int = 56
        eps: float = 1e-5
        decay: float = 0.75
        theta: float = 100.0
        device_parts: bool = False  # the variants of the toy parts that a captured decode step can hold
        architecture = "ToyHybridForCausalLM"

        @classmethod
        def from_dict(cls, raw):
            return cls(**{k: raw[k] for k in cls.__dataclass_fields__ if k in raw})

        def to_dict(self):
            return {**asdict(self), "architectures": [self.architecture], "model_type": "toy_hybrid"}

    def build_plan(cfg):
        H = cfg.hidden_size
        average = DeviceRunningAverageMixer if cfg.device_parts else RunningAverageMixer

        def attention(prefix, reads_only=False):
            return GQAttention(prefix, H, cfg.heads, cfg.kv_heads, cfg.head_dim,
                               NeighbourPairRotation(cfg.head_dim, cfg.theta, cfg.device_parts),
                               qk_norm_eps=cfg.eps, reads_only=reads_only)

        blocks = [
            Block(RMSNorm("b0.n1", H, cfg.eps), average("b0.gain", H, cfg.decay), RMSNorm("b0.n2", H, cfg.eps),
                  SwiGLU("b0.mlp.", H, cfg.inter)),
            Block(RMSNorm("b1.n1", H, cfg.eps), attention("b1.attn."), RMSNorm("b1.n2", H, cfg.eps),
                  TopOneOfTwo("b1.moe.", H, cfg.inter, cfg.device_parts)),
            Block(RMSNorm("b2.n1", H, cfg.eps), attention("b2.attn.", reads_only=True), None,
                  SwiGLU("b2.mlp.", H, cfg.inter), arrangement="parallel"),
        ]
        # block 0 runs twice (two state layers), block 2 reads the cache that block 1 filled
        order = [LayerCall(0, cache=0), LayerCall(1, cache=1), LayerCall(2, cache=1, write=False), LayerCall(0, cache=2)]
        return ModelPlan(Embedding("tok", cfg.vocab_size, H), blocks, order, RMSNorm("final", H, cfg.eps),
                         OutputHead("head", cfg.vocab_size, H), cfg.vocab_size, H, max_positions=512).validate()

    kirai_b200.register_architecture("ToyHybridForCausalLM", ToyConfig, build_plan, replace=True)
    return ToyConfig


def plain_toy_logits(cfg, w, tokens):
    """The toy model, whole sequence, on the CPU with plain arithmetic."""
    T, H, d = len(tokens), cfg.hidden_size, cfg.head_dim
    positions = torch.arange(T, dtype=torch.float32)

    def pair_rotation(x):
        half = d // 2
        freq = torch.pow(torch.tensor(cfg.theta), -torch.arange(half, dtype=torch.float32) / half)
        angle = positions[:, None, None] * freq[None, None, :]
        even, odd = x[..., 0::2], x[..., 1::2]
        out = torch.empty_like(x)
        out[..., 0::2] = even * torch.cos(angle) - odd * torch.sin(angle)
        out[..., 1::2] = odd * torch.cos(angle) + even * torch.sin(angle)
        return out

    def running_average(x, gain):
        state, rows = torch.zeros(H), []
        for t in range(T):
            state = cfg.decay * state + x[t]
            rows.append(state * gain)
        return torch.stack(rows)

    def mlp(x, prefix):
        return plain.swiglu_mlp(x, w[prefix + "gate_proj.weight"], w[prefix + "up_proj.weight"], w[prefix + "down_proj.weight"])

    def block0(h):
        r = h + running_average(plain.rms_norm(h, w["b0.n1"], cfg.eps), w["b0.gain"])
        return r + mlp(plain.rms_norm(r, w["b0.n2"], cfg.eps), "b0.mlp.")

    h = w["tok"][torch.tensor(tokens)]
    h = block0(h)
    # block 1: attention that fills the cache, routed feed-forward
    n = plain.rms_norm(h, w["b1.n1"], cfg.eps)
    q = pair_rotation(plain.rms_norm((n @ w["b1.attn.q_proj.weight"].T).reshape(T, cfg.heads, d), w["b1.attn.q_norm.weight"], cfg.eps))
    k = pair_rotation(plain.rms_norm((n @ w["b1.attn.k_proj.weight"].T).reshape(T, cfg.kv_heads, d), w["b1.attn.k_norm.weight"], cfg.eps))
    v = (n @ w["b1.attn.v_proj.weight"].T).reshape(T, cfg.kv_heads, d)
    r = h + plain.causal_attention(q, k, v, None).reshape(T, -1) @ w["b1.attn.o_proj.weight"].T
    n2 = plain.rms_norm(r, w["b1.n2"], cfg.eps)
    choice = (n2 @ w["b1.moe.router.weight"].T).argmax(-1)
    routed = torch.stack([mlp(n2[t : t + 1], f"b1.moe.experts.{int(choice[t])}.")[0] for t in range(T)])
    h = r + routed
    # block 2: its own queries over block 1's keys and values, parallel arrangement
    n = plain.rms_norm(h, w["b2.n1"], cfg.eps)
    q2 = pair_rotation(plain.rms_norm((n @ w["b2.attn.q_proj.weight"].T).reshape(T, cfg.heads, d), w["b2.attn.q_norm.weight"], cfg.eps))
    h = h + plain.causal_attention(q2, k, v, None).reshape(T, -1) @ w["b2.attn.o_proj.weight"].T + mlp(n, "b2.mlp.")
    h = block0(h)
    return plain.rms_norm(h, w["final"], cfg.eps) @ w["head"].T, choice


@pytest.mark.parametrize("dtype", DTYPES)
def test_toy_architecture_is_registered_built_and_stepped(dtype, tmp_path):
    ToyConfig = define_toys()
    from kirai_b200.engine.batch import StepEntry
    from kirai_b200.engine.runner import ModelRunner
    from kirai_b200.weights import write_random_model

    cfg = ToyConfig()
    write_random_model(str(tmp_path), cfg, seed=4, std=0.08)
    _, weights = plain.read_model_folder(str(tmp_path))
    runner = ModelRunner.from_folder(str(tmp_path), dtype=dtype, page_size=4, max_tokens=128, num_slots=3)
    assert type(runner.config).__name__ == "ToyConfig" and len(runner.cache.groups) == 1 and len(runner.cache.state) == 2
    sequences = {name: torch.randint(0, cfg.vocab_size, (n,), generator=torch.Generator().manual_seed(n)).tolist()
                 for name, n in (("a", 21), ("b", 9))}
    expected = {name: plain_toy_logits(cfg, weights, tokens) for name, tokens in sequences.items()}
    live = {name: runner.cache.open(name) for name in sequences}
    got = {name: [] for name in sequences}
    # a: 8 + 2 + 10 + 1 tokens; b joins in the second step with 5, then 3, then one decoded token
    plan = [[("a", 0, 8)], [("a", 8, 2), ("b", 0, 5)], [("a", 10, 10), ("b", 5, 3)], [("a", 20, 1), ("b", 8, 1)]]
    for step in plan:
        entries = [StepEntry(live[name], sequences[name][first : first + count], range(count)) for name, first, count in step]
        logits = runner.step(entries).cpu()
        row = 0
        for name, first, count in step:
            got[name].append(logits[row : row + count])
            row += count
    for name in sequences:
        reference, choice = expected[name]
        result = torch.cat(got[name])
        if dtype == torch.float32:
            assert float((result - reference).abs().max()) <= tolerance(dtype, reference)
        else:
            # a bf16 router may pick the other expert when its two logits are within rounding; compare where it cannot
            assert float((result[:4] - reference[:4]).abs().max()) <= 0.05 * float(reference.abs().max())
    for request in live.values():
        runner.cache.close(request)
    assert runner.cache.free_pages() == [32] and runner.cache.tables.slots.free_slots == 3
    # a fresh request in a reused slot starts from a zero state
    again = runner.cache.open("again")
    logits = runner.step([StepEntry(again, sequences["b"], range(9))]).cpu()
    if dtype == torch.float32:
        assert float((logits - expected["b"][0]).abs().max()) <= tolerance(dtype, expected["b"][0])


def plain_toy_generate(cfg, weights, prompt, params):
    """Token by token with the plain toy model and the plain sampler, and the engine's draws."""
    from kirai_b200.sampling import rng

    tokens, out = list(prompt), []
    for k in range(params.max_new_tokens):
        logits = plain_toy_logits(cfg, weights, tokens)[0][-1]
        if params.temperature == 0.0:
            out.append(plain.argmax_first(logits))
        else:
            out.append(plain.sample_top_p(logits, params.temperature, params.top_p, rng.draw(params.seed, k)))
        tokens.append(out[-1])
    return out


@pytest.mark.parametrize("device_parts", [False, True])
def test_toy_architecture_generates_through_the_engine(device_parts, tmp_path):
    """The toy architecture through ``Engine.generate``: scheduler, prompt portions, seeded sampling, a pool so small
    that a request which holds a state slot is evicted and recomputed, and CUDA graphs switched on.  With parts that
    walk requests on the host the engine must run every step eagerly; with parts that promise ``capture_safe`` it
    replays captured decode steps, and the state advances once per token either way."""
    ToyConfig = define_toys()
    from kirai_b200 import Engine, SamplingParams
    from kirai_b200.weights import write_random_model

    cfg = ToyConfig(device_parts=device_parts)
    write_random_model(str(tmp_path), cfg, seed=4, std=0.08)
    _, weights = plain.read_model_folder(str(tmp_path))
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=torch.Generator().manual_seed(70 + n)).tolist() for n in (9, 14, 6)]
    params = [SamplingParams(temperature=0.0, max_new_tokens=12),
              SamplingParams(temperature=0.8, top_p=0.9, seed=31, max_new_tokens=12),
              SamplingParams(temperature=1.1, top_p=1.0, seed=32, max_new_tokens=12)]
    expected = [plain_toy_generate(cfg, weights, prompt, p) for prompt, p in zip(prompts, params)]
    # 11 pages of 4 tokens: the three requests grow to 20, 25 and 17 tokens (5 + 7 + 5 pages), so one is evicted
    engine = Engine(str(tmp_path), dtype="float32", page_size=4, max_prefill_tokens=8, max_concurrent_requests=3,
                    max_new_tokens=12, max_cache_tokens=44, cuda_graphs=True)
    assert engine.runner.model.plan.capture_safe() is device_parts
    outputs = engine.generate(prompts, params)
    assert [o.token_ids for o in outputs] == expected
    stats = engine.stats()
    assert stats["scheduler"]["preemptions"] >= 1 and sum(o.preemptions for o in outputs) >= 1
    assert (stats["graph_steps"] > 0) is device_parts
    assert stats["cache"]["live_requests"] == 0 and all(g["used"] == 0 for g in stats["cache"]["groups"])
    # the same with every step eager
    eager = Engine(str(tmp_path), dtype="float32", page_size=4, max_prefill_tokens=8, max_concurrent_requests=3,
                   max_new_tokens=12, max_cache_tokens=44, cuda_graphs=False)
    assert [o.token_ids for o in eager.generate(prompts, params)] == expected


def test_a_captured_step_refuses_parts_that_read_host_lists(tmp_path):
    """A captured step's batch has no host copy of slots and start positions; a mixer that walks them (the toy's
    first form) must raise at capture, with a message that says what to do, never read a placeholder."""
    ToyConfig = define_toys()
    from kirai_b200.engine.graphs import DecodeGraph
    from kirai_b200.engine.runner import ModelRunner
    from kirai_b200.weights import write_random_model

    write_random_model(str(tmp_path), ToyConfig(), seed=4, std=0.08)
    runner = ModelRunner.from_folder(str(tmp_path), dtype="float32", page_size=4, max_tokens=64, num_slots=2)
    request = runner.cache.open("a")
    assert runner.cache.reserve(request, 1)
    graph = DecodeGraph(runner, 1, 16)
    graph.load_inputs([3], [0], [request.slot], [runner.cache.block_table_array([request], 0)], [0.0], [1.0], [0.5])
    with pytest.raises(RuntimeError, match="no host copy of batch.slot_ids"):
        graph.capture()
    torch.cuda.synchronize()


def test_plan_validation_refuses_bad_orders():
    define_toys()
    from kirai_b200.models.plan import LayerCall, PlanError
    from kirai_b200.registry import resolve

    config_class, build = resolve("ToyHybridForCausalLM")
    plan = build(config_class())
    for order in ([LayerCall(2, cache=0, write=False)],                       # read before any write
                  [LayerCall(1, cache=0), LayerCall(1, cache=0)],             # one cache layer written twice
                  [LayerCall(0, cache=0), LayerCall(1, cache=2)],             # a gap in the numbering
                  [LayerCall(5, cache=0)],                                    # no such block
                  [LayerCall(0, cache=0), LayerCall(2, cache=0, write=False)]):  # reader and cache of different kinds
        plan.order = order
        with pytest.raises(PlanError):
            plan.validate()
