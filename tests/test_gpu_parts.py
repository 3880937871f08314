"""Each part alone against the plain functions, a schedule that names a layer twice and
lets a layer read another layer's cache, and a toy mixer with state of its own that is
registered, built, loaded and stepped without a change to the package."""
import dataclasses

import numpy as np
import pytest
import torch

import plain_model
from tiny_configs import TINY_A

pytestmark = pytest.mark.gpu
DEVICE = torch.device("cuda:0")


def close(found, expected, tolerance, what=""):
    found, expected = found.double().cpu(), expected.double().cpu()
    error = float((found - expected).abs().max()) / max(1.0, float(expected.abs().max()))
    assert error <= tolerance, f"{what}: relative error {error:.3e} > {tolerance:.1e}"


def make_env(dtype, max_positions=512, positions=None):
    from kidi_b200.parts.base import BuildEnv
    from kidi_b200.parts.registry import build_part
    env = BuildEnv(dtype=dtype, device=DEVICE, max_positions=max_positions)
    for name, spec in (positions or {}).items():
        env.positions[name] = build_part("position", spec, env)
    return env


def random_tensors(part, dtype, seed=0):
    generator = torch.Generator().manual_seed(seed)
    tensors = {}
    for spec in part.parameter_specs():
        kind, std = spec.init
        values = torch.randn(spec.shape, generator=generator) * std + (1.0 if kind == "one_plus_normal" else 0.0)
        tensors[spec.name] = values.to(dtype)
    return tensors


def step_context(part_requests, starts, news, dtype, max_positions=512):
    """A cache for one schedule entry and the context of a step on fresh slots that
    already hold `starts[b]` tokens (their cache content is whatever earlier calls left)."""
    from kidi_b200.cache.sequence_cache import SequenceCache
    cache = SequenceCache([part_requests], max_tokens=4096, max_positions=max_positions, dtype=dtype, device=DEVICE)
    slots = [cache.acquire() for _ in starts]
    return cache, slots


def run_step(cache, slots, news_tokens, dtype):
    from kidi_b200.engine.engine import DeviceTables, StepContext
    from kidi_b200.engine.plan import StepBatch, build_plan
    starts = [cache.length(slot) for slot in slots]
    plan = build_plan(StepBatch(slots, news_tokens), starts, vocab_size=1 << 20)
    growth = [(slot, start + len(new)) for slot, start, new in zip(slots, starts, news_tokens)]
    cache.reserve(growth)
    cache.flush_tables()
    buffer = torch.from_numpy(plan.packed()).to(DEVICE)
    ctx = StepContext(plan, DeviceTables(buffer, plan.offsets()), cache, dtype, DEVICE)
    return ctx, growth


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_part_takes_the_pending_delta(dtype):
    from kidi_b200.parts.base import ResidualStream
    from kidi_b200.parts.registry import build_part
    from kidi_b200.parts.spec import PartSpec
    env = make_env(dtype)
    norm = build_part("norm", PartSpec("rms_norm", {"size": 200, "eps": 1e-5}), env)
    tensors = random_tensors(norm, dtype)
    norm.bind({name: t.to(DEVICE) for name, t in tensors.items()})
    hidden = torch.randn(9, 200, generator=torch.Generator().manual_seed(1))
    delta = torch.randn(9, 200, generator=torch.Generator().manual_seed(2)).to(dtype)
    stream = ResidualStream(hidden.to(DEVICE))
    stream.add(delta.to(DEVICE))
    out = norm.forward(stream)
    assert stream.pending is None and out.dtype == dtype
    summed = hidden.double() + delta.double()
    close(stream.hidden, summed, 1e-6)
    close(out, plain_model.rms_norm(summed, tensors["weight"].double(), 1e-5), 1e-5 if dtype == torch.float32 else 8e-3)


def test_embedding_and_head_parts():
    from kidi_b200.parts.registry import build_part
    from kidi_b200.parts.spec import PartSpec
    env = make_env(torch.bfloat16)
    embedding = build_part("embedding", PartSpec("token_embedding", {"vocab_size": 301, "hidden_size": 72, "scale": 1.0}), env)
    table = random_tensors(embedding, torch.bfloat16)["weight"]
    embedding.bind({"weight": table.to(DEVICE)})
    tokens = torch.tensor([0, 300, 5, 5], dtype=torch.int32)
    out = embedding.forward(tokens.to(DEVICE), None)
    assert torch.equal(out.cpu(), plain_model.embed(tokens.tolist(), table))
    head = build_part("head", PartSpec("linear_head", {"vocab_size": 301, "hidden_size": 72, "tied_to": None}), env)
    head.bind({"weight": table.to(DEVICE)})
    x = torch.randn(70, 72, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16)
    logits = head.forward(x.to(DEVICE), None)
    assert logits.dtype == torch.float32
    close(logits, x.double() @ table.double().T, 2e-5, "head, many rows")       # 32-bit logits from bfloat16 operands
    close(head.forward(x[:3].to(DEVICE), None), x[:3].double() @ table.double().T, 2e-5, "head, few rows")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows", [5, 100])
def test_feed_forward_part(dtype, rows):
    from kidi_b200.parts.registry import build_part
    from kidi_b200.parts.spec import PartSpec
    env = make_env(dtype)
    part = build_part("feed_forward", PartSpec("gated_mlp", {"hidden_size": 96, "intermediate_size": 200,
                                                             "activation": "silu"}, "mlp."), env)
    tensors = random_tensors(part, dtype, seed=4)
    tensors = {name: t * 5 for name, t in tensors.items()}          # large enough for the gate to bend
    part.bind({name: t.to(DEVICE) for name, t in tensors.items()})
    x = torch.randn(rows, 96, generator=torch.Generator().manual_seed(5)).to(dtype)
    unfused = {"mlp.gate_proj.weight": tensors["gate_up_proj.weight"][:200], "mlp.up_proj.weight": tensors["gate_up_proj.weight"][200:],
               "mlp.down_proj.weight": tensors["down_proj.weight"]}
    expected = plain_model.gated_feed_forward(x.double(), unfused, "mlp.")
    close(part.forward(x.to(DEVICE), None), expected, 2e-6 if dtype == torch.float32 else 2e-2, "gated mlp")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [None, 40])
def test_attention_part_prompt_then_tokens(dtype, window):
    """The mixer alone: a prompt, then single tokens, against the plain layer on whole sequences."""
    from kidi_b200.parts.registry import build_part
    from kidi_b200.parts.spec import PartSpec
    hidden, heads, kv_heads, width = 80, 6, 2, 48
    rope = PartSpec("rotary", {"head_dim": width, "rotary_dim": width, "theta": 5e4, "max_positions": 512})
    env = make_env(dtype, positions={"rope": rope})
    part = build_part("mixer", PartSpec("attention", {
        "hidden_size": hidden, "num_heads": heads, "num_kv_heads": kv_heads, "head_dim": width, "qk_norm": True,
        "qk_norm_eps": 1e-6, "position": "rope", "window": window}, "attn."), env)
    tensors = {name: t * (8 if "proj" in name else 1) for name, t in random_tensors(part, dtype, seed=6).items()}
    part.bind({name: t.to(DEVICE) for name, t in tensors.items()})
    lengths = [150, 70]
    x = [torch.randn(n, hidden, generator=torch.Generator().manual_seed(10 + n)).to(dtype) for n in lengths]
    q_rows, kv_rows = heads * width, kv_heads * width
    fused = tensors["qkv_proj.weight"]
    plain_tensors = {"attn.q_proj.weight": fused[:q_rows], "attn.k_proj.weight": fused[q_rows:q_rows + kv_rows],
                     "attn.v_proj.weight": fused[q_rows + kv_rows:], "attn.o_proj.weight": tensors["o_proj.weight"],
                     "attn.q_norm.weight": tensors["q_norm.weight"], "attn.k_norm.weight": tensors["k_norm.weight"]}
    config = {"num_attention_heads": heads, "num_key_value_heads": kv_heads, "head_dim": width, "rms_norm_eps": 1e-6}
    expected = []
    for sequence in x:
        cos, sin = plain_model.rotary_tables(sequence.shape[0], width, 5e4)
        expected.append(plain_model.attention_layer(sequence.double(), plain_tensors, "attn.", config, cos, sin, window))
    cache, slots = step_context(part.cache_requests(), [0, 0], None, dtype)
    heads_first = [100, 69]
    ctx, growth = run_step(cache, slots, [[0] * n for n in heads_first], dtype)
    out = part.forward(torch.cat([x[0][:100], x[1][:69]]).to(DEVICE), ctx, cache.views(0), True)
    cache.commit(growth)
    tolerance = 5e-6 if dtype == torch.float32 else 3e-2
    close(out[:100], expected[0][:100], tolerance, "prompt 0")
    close(out[100:], expected[1][:69], tolerance, "prompt 1")
    for step in range(50):
        live = [b for b in range(2) if heads_first[b] + step < lengths[b]]
        ctx, growth = run_step(cache, [slots[b] for b in live], [[0] for _ in live], dtype)
        rows = torch.stack([x[b][heads_first[b] + step] for b in live]).to(DEVICE)
        out = part.forward(rows, ctx, cache.views(0), True)
        cache.commit(growth)
        for index, b in enumerate(live):
            close(out[index], expected[b][heads_first[b] + step], tolerance, f"sequence {b}, token {heads_first[b] + step}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_part_with_biases(dtype):
    """The same mixer with a bias on the fused q/k/v projection (bound from q, k and v biases by
    the loader's concatenation rule) and on the output projection: prompts of 5 and 150 rows
    (the few-row and the many-row products), then single tokens."""
    from kidi_b200.parts.base import all_parameters
    from kidi_b200.parts.registry import build_part
    from kidi_b200.parts.spec import PartSpec
    from kidi_b200.weights.loader import TensorDict, bind_parameters
    hidden, heads, kv_heads, width = 64, 4, 2, 32
    rope = PartSpec("rotary", {"head_dim": width, "rotary_dim": width, "theta": 1e4, "max_positions": 512})
    env = make_env(dtype, positions={"rope": rope})
    part = build_part("mixer", PartSpec("attention", {
        "hidden_size": hidden, "num_heads": heads, "num_kv_heads": kv_heads, "head_dim": width, "qk_norm": True,
        "qk_norm_eps": 1e-6, "position": "rope", "window": None, "qkv_bias": True, "out_bias": True}, "attn."), env)
    generator = torch.Generator().manual_seed(21)
    draw = lambda *shape, scale=1.0: (torch.randn(*shape, generator=generator) * scale).to(dtype)
    q_rows, kv_rows = heads * width, kv_heads * width
    stored = {"attn.q_proj.weight": draw(q_rows, hidden, scale=0.15), "attn.k_proj.weight": draw(kv_rows, hidden, scale=0.15),
              "attn.v_proj.weight": draw(kv_rows, hidden, scale=0.15), "attn.o_proj.weight": draw(hidden, q_rows, scale=0.15),
              "attn.q_proj.bias": draw(q_rows), "attn.k_proj.bias": draw(kv_rows), "attn.v_proj.bias": draw(kv_rows),
              "attn.o_proj.bias": draw(hidden), "attn.q_norm.weight": 1 + draw(width, scale=0.1),
              "attn.k_norm.weight": 1 + draw(width, scale=0.1)}
    bound = bind_parameters(all_parameters(part), TensorDict(stored), engine_dtype=dtype, device=DEVICE)
    assert bound["attn.qkv_proj.bias"].shape == (q_rows + 2 * kv_rows,)
    part.bind({name[len("attn."):]: tensor for name, tensor in bound.items()})

    def plain(x):                                    # the plain layer's steps with the biases added
        length = x.shape[0]
        w = lambda name: stored["attn." + name].double()
        cos, sin = plain_model.rotary_tables(length, width, 1e4)
        q = (x @ w("q_proj.weight").T + w("q_proj.bias")).reshape(length, heads, width)
        k = (x @ w("k_proj.weight").T + w("k_proj.bias")).reshape(length, kv_heads, width)
        v = (x @ w("v_proj.weight").T + w("v_proj.bias")).reshape(length, kv_heads, width)
        q = plain_model.norm_then_rotate(q, w("q_norm.weight"), 1e-6, cos, sin)
        k = plain_model.norm_then_rotate(k, w("k_norm.weight"), 1e-6, cos, sin)
        return plain_model.causal_attention(q, k, v) @ w("o_proj.weight").T + w("o_proj.bias")

    lengths, heads_first = [160, 12], [150, 5]
    x = [torch.randn(n, hidden, generator=generator).to(dtype) for n in lengths]
    expected = [plain(sequence.double()) for sequence in x]
    cache, slots = step_context(part.cache_requests(), [0, 0], None, dtype)
    ctx, growth = run_step(cache, slots, [[0] * n for n in heads_first], dtype)
    out = part.forward(torch.cat([x[0][:150], x[1][:5]]).to(DEVICE), ctx, cache.views(0), True)
    cache.commit(growth)
    tolerance = 5e-6 if dtype == torch.float32 else 2e-2
    close(out[:150], expected[0][:150], tolerance, "prompt 0 with biases")
    close(out[150:], expected[1][:5], tolerance, "prompt 1 with biases")
    for step in range(7):
        ctx, growth = run_step(cache, slots, [[0], [0]], dtype)
        rows = torch.stack([x[b][heads_first[b] + step] for b in range(2)]).to(DEVICE)
        out = part.forward(rows, ctx, cache.views(0), True)
        cache.commit(growth)
        for b in range(2):
            close(out[b], expected[b][heads_first[b] + step], tolerance, f"sequence {b}, token {heads_first[b] + step}")


# ------------------------------------------------- schedules: a layer twice, a shared cache
def test_schedule_names_a_layer_twice_and_shares_a_cache(tmp_path):
    """The run order is data: [0, 1, 0] runs layer 0 twice (each run with a cache of its
    own); with `cache_from` the third entry reads the first entry's cache instead."""
    from kidi_b200 import Engine, StepBatch, register_architecture, write_random_model
    from kidi_b200.config.qwen3 import Qwen3Config
    from kidi_b200.models import qwen3
    from kidi_b200.parts.spec import ScheduleEntry

    def twice(config):
        return dataclasses.replace(qwen3.build_spec(config), architecture="TwiceForCausalLM",
                                   schedule=(ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0)))

    def shared(config):
        return dataclasses.replace(qwen3.build_spec(config), architecture="SharedForCausalLM",
                                   schedule=(ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0, cache_from=0)))

    register_architecture("TwiceForCausalLM", Qwen3Config, twice)
    register_architecture("SharedForCausalLM", Qwen3Config, shared)
    tokens = np.random.default_rng(0).integers(0, 256, size=90).tolist()
    folder = write_random_model(dict(TINY_A, architectures=["TwiceForCausalLM"]), str(tmp_path / "twice"), seed=3)
    config, tensors = plain_model.read_model_folder(folder)
    expected = plain_model.forward(config, tensors, tokens, schedule=[0, 1, 0]).numpy()
    engine = Engine.load(folder, dtype="float32")
    assert engine.cache.kv_groups[0].keys.shape[0] == 3               # three entries, three caches
    slot = engine.acquire()
    first = engine.step(StepBatch([slot], [tokens[:60]], [list(range(60))])).cpu().numpy()
    rest = [engine.step(StepBatch([slot], [[t]], [[0]])).cpu().numpy() for t in tokens[60:]]
    found = np.concatenate([first, *rest])
    assert np.abs(found - expected).max() <= 2e-5 * max(1.0, np.abs(expected).max())

    # Sharing: the third entry attends over the FIRST entry's keys and values with its own queries.
    folder = write_random_model(dict(TINY_A, architectures=["SharedForCausalLM"]), str(tmp_path / "shared"), seed=3)
    engine = Engine.load(folder, dtype="float32")
    assert engine.cache.kv_groups[0].keys.shape[0] == 2               # the third entry owns no storage
    slot = engine.acquire()
    whole = engine.step(StepBatch([slot], [tokens], [list(range(90))])).cpu().numpy()
    engine.release(slot)
    slot = engine.acquire()
    parts = [engine.step(StepBatch([slot], [tokens[:50]], [list(range(50))])).cpu().numpy()]
    parts += [engine.step(StepBatch([slot], [[t]], [[0]])).cpu().numpy() for t in tokens[50:]]
    assert np.array_equal(np.concatenate(parts), whole)                # the same under every cut
    assert np.abs(whole - expected).max() > 1e-3                       # and not the unshared model


# -------------------------------------------- a toy mixer with state of its own
def plain_toy_forward(config, tensors, tokens):
    """The toy model on a whole sequence: layer 0 mixes with s_t = decay * s_{t-1} + x_t W,
    layer 1 with attention; both keep the usual norms and feed-forward."""
    dtype = torch.float64
    hidden = plain_model.embed(tokens, tensors["model.embed_tokens.weight"], dtype)
    cos, sin = plain_model.rotary_tables(len(tokens), config["head_dim"], config["rope_theta"])
    eps = config["rms_norm_eps"]
    for layer in range(2):
        prefix = f"model.layers.{layer}."
        normed = plain_model.rms_norm(hidden, tensors[prefix + "input_layernorm.weight"], eps)
        if layer == 0:
            projected = normed @ tensors[prefix + "mixer.in_proj.weight"].to(dtype).T
            state = torch.zeros(config["hidden_size"], dtype=dtype)
            mixed = torch.empty_like(projected)
            for t in range(len(tokens)):
                state = config["decay"] * state + projected[t]
                mixed[t] = state
        else:
            mixed = plain_model.attention_layer(normed, tensors, prefix + "self_attn.", config, cos, sin, None)
        hidden = hidden + mixed
        hidden = hidden + plain_model.gated_feed_forward(
            plain_model.rms_norm(hidden, tensors[prefix + "post_attention_layernorm.weight"], eps), tensors, prefix + "mlp.")
    hidden = plain_model.rms_norm(hidden, tensors["model.norm.weight"], eps)
    return (hidden @ tensors["lm_head.weight"].to(dtype).T).float().numpy()


def test_a_toy_mixer_with_state_of_its_own(tmp_path):
    from kidi_b200 import Engine, StepBatch, register_architecture, register_part, write_random_model
    from kidi_b200.cache.sequence_cache import StateRequest
    from kidi_b200.config.qwen3 import Qwen3Config
    from kidi_b200.models import qwen3
    from kidi_b200.parts.base import Part
    from kidi_b200.parts.spec import LayerSpec, ParamSpec, PartSpec

    @register_part("mixer", "toy_decay")
    class ToyDecayMixer(Part):
        """s_t = decay * s_{t-1} + x_t W; y_t = s_t. The state is one vector per sequence."""

        def __init__(self, spec, env):
            super().__init__(spec, env)
            self.hidden, self.decay = int(spec.param("hidden_size")), float(spec.param("decay"))

        def parameter_specs(self):
            return [ParamSpec("in_proj.weight", (self.hidden, self.hidden), init=("normal", 0.1))]

        def bind(self, tensors):
            self.weight = tensors["in_proj.weight"]

        def cache_requests(self):
            return [StateRequest((self.hidden,), torch.float32)]

        def forward(self, x, ctx, views, owns_cache):
            state = views[0]                                  # [slots + 1, hidden]; the last row is the padding slot's
            projected = x.float() @ self.weight.float().T
            plan = ctx.plan
            if plan.is_decode:
                # One token per sequence, row b for sequence b: from the device tables alone, so
                # that a captured step can replay it. Padding sequences of such a step carry the
                # padding slot: their (meaningless) state lands in the last row.
                slot = ctx.tables.seq_slot.long()
                current = self.decay * state[slot] + projected
                state.index_copy_(0, slot, current)
                return current.to(x.dtype)
            out = torch.empty_like(projected)
            for b in range(plan.n_seqs):
                slot, row0, count = int(plan.seq_slot[b]), int(plan.seq_row0[b]), int(plan.seq_len[b])
                current = state[slot].clone()
                for t in range(count):
                    current = self.decay * current + projected[row0 + t]
                    out[row0 + t] = current
                state[slot] = current
            return out.to(x.dtype)

    @dataclasses.dataclass(frozen=True)
    class ToyConfig:
        base: Qwen3Config
        decay: float

        @classmethod
        def from_dict(cls, values):
            return cls(Qwen3Config.from_dict({k: v for k, v in values.items() if k != "decay"}), float(values["decay"]))

    def build(config):
        spec = qwen3.build_spec(config.base)
        first = spec.layers[0]
        parts = dict(first.parts)
        parts["mixer"] = PartSpec("toy_decay", {"hidden_size": config.base.hidden_size, "decay": config.decay},
                                  "model.layers.0.mixer.")
        layers = (LayerSpec(first.arrangement, parts), *spec.layers[1:])
        return dataclasses.replace(spec, architecture="ToyDecayForCausalLM", layers=layers)

    register_architecture("ToyDecayForCausalLM", ToyConfig, build)
    raw = dict(TINY_A, architectures=["ToyDecayForCausalLM"], decay=0.9, tie_word_embeddings=False)
    folder = write_random_model(raw, str(tmp_path / "toy"), seed=9, dtype=torch.float32)
    config, tensors = plain_model.read_model_folder(folder)
    assert "model.layers.0.mixer.in_proj.weight" in tensors and "model.layers.0.self_attn.q_proj.weight" not in tensors
    engine = Engine.load(folder, dtype="float32", max_tokens=256)
    assert len(engine.cache.state_groups) == 1 and len(engine.cache.kv_groups) == 1
    assert engine.cache.kv_groups[0].keys.shape[0] == 1               # only the attention layer keeps keys
    generator = np.random.default_rng(2)
    requests = [generator.integers(0, 256, size=n).tolist() for n in (40, 17, 64)]
    expected = [plain_toy_forward(config, tensors, tokens) for tokens in requests]
    # A batch of unequal prompts, then one token each; then a third request on a slot that was used before.
    slots = [engine.acquire(), engine.acquire()]
    heads = [25, 9]
    logits = engine.step(StepBatch(slots, [requests[0][:25], requests[1][:9]], [list(range(25)), list(range(9))])).cpu().numpy()
    found = [[logits[:25]], [logits[25:]]]
    done = list(heads)
    while any(done[b] < len(requests[b]) for b in range(2)):
        live = [b for b in range(2) if done[b] < len(requests[b])]
        logits = engine.step(StepBatch([slots[b] for b in live], [[requests[b][done[b]]] for b in live],
                                       [[0] for _ in live])).cpu().numpy()
        for index, b in enumerate(live):
            found[b].append(logits[index:index + 1])
            done[b] += 1
    for b in range(2):
        got = np.concatenate(found[b])
        assert np.abs(got - expected[b]).max() <= 5e-5 * max(1.0, np.abs(expected[b]).max()), b
        engine.release(slots[b])
    slot = engine.acquire()                                              # a used slot: its state starts from zero
    got = engine.step(StepBatch([slot], [requests[2]], [list(range(64))])).cpu().numpy()
    assert np.abs(got - expected[2]).max() <= 5e-5 * max(1.0, np.abs(expected[2]).max())
    engine.release(slot)
    engine.cache.check()

    # The same mixer inside the replayed decode graph, with a padding row: a bystander holds slot 0
    # and keeps its state there while three other sequences decode in a captured step of four
    # rows. The fourth row is padding; it carries the cache's padding slot, not slot 0, so the
    # bystander's state is what its own tokens made it.
    from kidi_b200.engine.decode_graph import DecodeSession
    from kidi_b200.sampling.sampler import Sampler
    taken = [engine.acquire(), engine.acquire()]
    bystander = 0                                   # the slot a padding sequence must never stand for
    assert bystander in taken
    engine.release(taken[1 - taken.index(bystander)])
    engine.step(StepBatch([bystander], [requests[2][:30]], [[]]))
    others = [generator.integers(0, 256, size=n).tolist() for n in (12, 20, 33)]
    wanted = [plain_toy_forward(config, tensors, tokens) for tokens in others]
    slots = [engine.acquire() for _ in others]
    heads = [len(tokens) - 6 for tokens in others]
    engine.step(StepBatch(slots, [tokens[:head] for tokens, head in zip(others, heads)], [[], [], []]))
    session = DecodeSession(engine, 4, Sampler(0), longest=64)
    session.load(slots, [tokens[head] for tokens, head in zip(others, heads)], [0.0] * 3, [0, 1, 2], [1] * 3)
    for step in range(6):
        session.step([tokens[head + step] for tokens, head in zip(others, heads)])
        logits = session.logits[:3].cpu().numpy()
        for b in range(3):
            reference = wanted[b][heads[b] + step]
            assert np.abs(logits[b] - reference).max() <= 5e-5 * max(1.0, np.abs(reference).max()), (b, step)
    after = engine.step(StepBatch([bystander], [requests[2][30:]], [list(range(34))])).cpu().numpy()
    assert np.abs(after - expected[2][30:]).max() <= 5e-5 * max(1.0, np.abs(expected[2]).max()), \
        "a padding row of the captured step changed the state of a sequence outside it"
    assert engine.cache.padding_slot == engine.cache.n_slots
    for held in [bystander, *slots]:
        engine.release(held)
    engine.cache.check()
