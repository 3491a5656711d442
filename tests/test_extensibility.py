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
from part_helpers import DEV, tolerance

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

    class NeighbourPairRotation(PositionEncoding):
        """Rotates the pairs (2i, 2i + 1) by position * theta^(-i / (d/2)): another pairing than the half split."""

        def __init__(self, head_dim, theta):
            self.head_dim, self.theta = head_dim, theta

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

        def __init__(self, prefix, hidden, inter):
            self.router = Linear([(prefix + "router.weight", 2)], hidden)
            self.experts = [SwiGLU(prefix + f"experts.{e}.", hidden, inter) for e in range(2)]

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
        architecture = "ToyHybridForCausalLM"

        @classmethod
        def from_dict(cls, raw):
            return cls(**{k: raw[k] for k in cls.__dataclass_fields__ if k in raw})

        def to_dict(self):
            return {**asdict(self), "architectures": [self.architecture], "model_type": "toy_hybrid"}

    def build_plan(cfg):
        H = cfg.hidden_size

        def attention(prefix, reads_only=False):
            return GQAttention(prefix, H, cfg.heads, cfg.kv_heads, cfg.head_dim, NeighbourPairRotation(cfg.head_dim, cfg.theta),
                               qk_norm_eps=cfg.eps, reads_only=reads_only)

        blocks = [
            Block(RMSNorm("b0.n1", H, cfg.eps), RunningAverageMixer("b0.gain", H, cfg.decay), RMSNorm("b0.n2", H, cfg.eps),
                  SwiGLU("b0.mlp.", H, cfg.inter)),
            Block(RMSNorm("b1.n1", H, cfg.eps), attention("b1.attn."), RMSNorm("b1.n2", H, cfg.eps),
                  TopOneOfTwo("b1.moe.", H, cfg.inter)),
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


def test_plan_validation_refuses_bad_orders():
    define_toys()
    from kirai_b200.models.plan import LayerCall, PlanError
    from kirai_b200.registry import plan_for_config, resolve

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
