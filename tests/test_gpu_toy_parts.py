"""Parts of other kinds than the package has, defined here and registered from outside:
a feed-forward that routes every token to two of four small experts, a position table
that is added to the embeddings, a rotary encoding of half the head with slowed
positions, a norm that subtracts the mean and has a bias, and a block that runs mixer and
feed-forward side by side. Each is built from a specification, given random weights through the
package's own writer, loaded by tensor name and stepped through the engine (whole
requests, chunks, batches of unequal lengths, single tokens) against a plain model
written here. They are toys: no model of anyone's.
"""
import dataclasses

import numpy as np
import pytest
import torch

import plain_model
import replay_helpers as rh
from tiny_configs import sharpen_logits

pytestmark = pytest.mark.gpu

# Relative to the largest logit (the final norm is scaled so that it is 5 to 10): three times
# what was measured on a B200.
FP32_TOLERANCE = 1e-5
BF16_TOLERANCE = 2.5e-2

# Two layers, 3 heads over one key/value head, head width 64 (the tensor-core kernels'
# narrowest width, so that the bfloat16 run takes them), odd vocabulary.
BASE = {
    "model_type": "qwen3", "hidden_act": "silu", "num_hidden_layers": 2, "hidden_size": 80,
    "num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 64, "intermediate_size": 120,
    "vocab_size": 203, "rope_theta": 10000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False,
    "max_position_embeddings": 320,
}


def wrapped_config(extra_keys):
    """A configuration type that reads the base keys as a Qwen3Config and keeps `extra_keys`."""
    from kidi_b200.config.qwen3 import Qwen3Config

    @dataclasses.dataclass(frozen=True)
    class Wrapped:
        base: Qwen3Config
        extra: dict

        @classmethod
        def from_dict(cls, values):
            base = {key: value for key, value in values.items() if key not in extra_keys}
            return cls(Qwen3Config.from_dict(base), {key: values[key] for key in extra_keys})

    return Wrapped


def plain_layers(config, tensors, tokens, mixers, feed_forwards, on_embeddings=None):
    """The pre-norm model on a whole sequence with a given mixer and feed-forward per layer."""
    dtype = torch.float64
    hidden = plain_model.embed(tokens, tensors["model.embed_tokens.weight"], dtype)
    if on_embeddings is not None:
        hidden = on_embeddings(hidden)
    eps = config["rms_norm_eps"]
    for layer, (mixer, feed_forward) in enumerate(zip(mixers, feed_forwards)):
        prefix = f"model.layers.{layer}."
        hidden = hidden + mixer(plain_model.rms_norm(hidden, tensors[prefix + "input_layernorm.weight"], eps), prefix)
        hidden = hidden + feed_forward(
            plain_model.rms_norm(hidden, tensors[prefix + "post_attention_layernorm.weight"], eps), prefix)
    hidden = plain_model.rms_norm(hidden, tensors["model.norm.weight"], eps)
    return (hidden @ tensors["lm_head.weight"].to(dtype).T).float().numpy()


def run_every_way(engine, requests, expected, tolerance, what):
    rh.assert_matches(rh.run_whole(engine, requests), expected, tolerance, what + ", whole")
    rh.assert_matches(rh.run_tail_decoded(engine, requests, 32), expected, tolerance, what + ", last 32 one by one")
    rh.assert_matches(rh.run_batches(engine, requests, batch_size=3), expected, tolerance, what + ", batches of 3")
    rh.assert_matches(rh.run_chunked(engine, requests, chunk=100), expected, tolerance, what + ", chunks of 100")
    engine.cache.check()
    assert not engine.cache.slots.held


# ------------------------------------------------------- a feed-forward with routing
def test_a_toy_feed_forward_with_routing(tmp_path):
    from kidi_b200 import Engine, register_architecture, register_part, write_random_model
    from kidi_b200.models import qwen3
    from kidi_b200.parts.base import Part
    from kidi_b200.parts.spec import LayerSpec, ParamSpec, PartSpec

    @register_part("feed_forward", "toy_routed")
    class ToyRoutedFeedForward(Part):
        """Router logits in 32-bit; the `top` largest choose the experts, a softmax over those
        logits weighs them; every expert is a small SiLU-gated feed-forward."""

        def __init__(self, spec, env):
            super().__init__(spec, env)
            self.hidden, self.inter = int(spec.param("hidden_size")), int(spec.param("intermediate_size"))
            self.experts, self.top = int(spec.param("experts")), int(spec.param("top"))

        def parameter_specs(self):
            return [ParamSpec("router.weight", (self.experts, self.hidden), init=("normal", 1.0)),
                    ParamSpec("experts.gate_up_proj.weight", (self.experts, 2 * self.inter, self.hidden), init=("normal", 0.2)),
                    ParamSpec("experts.down_proj.weight", (self.experts, self.hidden, self.inter), init=("normal", 0.2))]

        def bind(self, tensors):
            self.router = tensors["router.weight"]
            self.gate_up = tensors["experts.gate_up_proj.weight"]
            self.down = tensors["experts.down_proj.weight"]

        def forward(self, x, ctx):
            rows = x.float()
            logits = rows @ self.router.float().T
            values, chosen = logits.topk(self.top, dim=-1)
            share = torch.zeros_like(logits).scatter_(1, chosen, torch.softmax(values, dim=-1))
            out = torch.zeros_like(rows)
            for expert in range(self.experts):
                both = rows @ self.gate_up[expert].float().T
                gate, up = both[:, :self.inter], both[:, self.inter:]
                out += share[:, expert:expert + 1] * ((gate / (1.0 + torch.exp(-gate)) * up) @ self.down[expert].float().T)
            return out.to(x.dtype)

    Config = wrapped_config(("experts", "experts_top", "expert_size"))

    def build(config):
        spec = qwen3.build_spec(config.base)
        last = spec.layers[1]
        parts = dict(last.parts)
        parts["feed_forward"] = PartSpec("toy_routed", {
            "hidden_size": config.base.hidden_size, "intermediate_size": config.extra["expert_size"],
            "experts": config.extra["experts"], "top": config.extra["experts_top"]}, "model.layers.1.routed.")
        return dataclasses.replace(spec, architecture="ToyRoutedForCausalLM",
                                   layers=(spec.layers[0], LayerSpec(last.arrangement, parts)))

    register_architecture("ToyRoutedForCausalLM", Config, build)
    raw = dict(BASE, architectures=["ToyRoutedForCausalLM"], experts=4, experts_top=2, expert_size=24)
    folder = write_random_model(raw, str(tmp_path / "routed"), seed=21, dtype=torch.float32)
    sharpen_logits(folder)
    config, tensors = plain_model.read_model_folder(folder)
    assert tensors["model.layers.1.routed.experts.down_proj.weight"].shape == (4, 80, 24)
    assert "model.layers.1.mlp.down_proj.weight" not in tensors and "model.layers.0.mlp.down_proj.weight" in tensors
    cos, sin = plain_model.rotary_tables(config["max_position_embeddings"], config["head_dim"], config["rope_theta"])
    margins = []

    def attention(x, prefix):
        n = x.shape[0]
        return plain_model.attention_layer(x, tensors, prefix + "self_attn.", config, cos[:n], sin[:n], None)

    def dense(x, prefix):
        return plain_model.gated_feed_forward(x, tensors, prefix + "mlp.")

    def routed(x, prefix):
        w = lambda name: tensors[prefix + "routed." + name].double()
        logits = x @ w("router.weight").T
        ordered = logits.sort(dim=-1, descending=True).values
        margins.append(float((ordered[:, 1] - ordered[:, 2]).min()))
        out = torch.zeros_like(x)
        for row in range(x.shape[0]):
            chosen = torch.argsort(logits[row], descending=True)[:2]
            share = torch.softmax(logits[row, chosen], dim=0)
            for weight, expert in zip(share, chosen.tolist()):
                both = w("experts.gate_up_proj.weight")[expert] @ x[row]
                gate, up = both[:24], both[24:]
                out[row] += weight * (w("experts.down_proj.weight")[expert] @ (gate / (1.0 + torch.exp(-gate)) * up))
        return out

    requests = rh.random_requests(config["vocab_size"], [5, 70, 131, 200], seed=22)
    expected = {name: plain_layers(config, tensors, tokens, [attention, attention], [dense, routed])
                for name, tokens in requests.items()}
    assert min(margins) > 1e-4, "a token sits on the edge between two experts: take another seed"
    engine = Engine.load(folder, dtype="float32", max_tokens=1024)
    run_every_way(engine, requests, expected, FP32_TOLERANCE, "routed feed-forward")


# ------------------------------------------------------------ other position encodings
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_position_encodings(tmp_path, dtype):
    from kidi_b200 import Engine, register_architecture, register_part, write_random_model
    from kidi_b200.models import qwen3
    from kidi_b200.parts.base import Part
    from kidi_b200.parts.spec import LayerSpec, ParamSpec, PartSpec

    @register_part("position", "toy_table")
    class ToyPositionTable(Part):
        """A learned vector per position, added to the embeddings; mixers read nothing from it."""

        def __init__(self, spec, env):
            super().__init__(spec, env)
            self.size, self.hidden = int(spec.param("max_positions")), int(spec.param("hidden_size"))

        def parameter_specs(self):
            return [ParamSpec("weight", (self.size, self.hidden), init=("normal", 0.05))]

        def bind(self, tensors):
            self.table = tensors["weight"]

        def on_embeddings(self, stream, ctx):
            stream.hidden += self.table[ctx.tables.row_pos.long()].float()

    @register_part("position", "toy_slow_rotary")
    class ToySlowRotary(Part):
        """Rotates the first `rotary_dim` elements of a head by angles of position / factor."""

        def __init__(self, spec, env):
            super().__init__(spec, env)
            self.head_dim, self.rotary_dim = int(spec.param("head_dim")), int(spec.param("rotary_dim"))
            half = self.rotary_dim // 2
            frequency = 1.0 / torch.pow(torch.tensor(float(spec.param("theta"))),
                                        2.0 * torch.arange(half, dtype=torch.float32) / self.rotary_dim)
            angle = (torch.arange(int(spec.param("max_positions")), dtype=torch.float32)
                     / float(spec.param("factor")))[:, None] * frequency[None, :]
            self.cos, self.sin = torch.cos(angle).to(env.device), torch.sin(angle).to(env.device)

        def on_embeddings(self, stream, ctx):
            return None

    Config = wrapped_config(("slow_factor", "slow_width"))

    def build(config):
        base = config.base
        spec = qwen3.build_spec(base)
        layers = []
        for index, (layer, position) in enumerate(zip(spec.layers, (None, "slow"))):
            parts = dict(layer.parts)
            mixer = parts["mixer"]
            parts["mixer"] = PartSpec(mixer.kind, dict(mixer.params, position=position), mixer.prefix)
            layers.append(LayerSpec(layer.arrangement, parts))
        positions = {
            "table": PartSpec("toy_table", {"max_positions": base.max_position_embeddings,
                                            "hidden_size": base.hidden_size}, "model.position_table."),
            "slow": PartSpec("toy_slow_rotary", {"head_dim": base.head_dim, "rotary_dim": config.extra["slow_width"],
                                                 "theta": base.rope_theta, "factor": config.extra["slow_factor"],
                                                 "max_positions": base.max_position_embeddings}),
        }
        return dataclasses.replace(spec, architecture="ToyPositionsForCausalLM", layers=tuple(layers), positions=positions)

    register_architecture("ToyPositionsForCausalLM", Config, build)
    raw = dict(BASE, architectures=["ToyPositionsForCausalLM"], slow_factor=4.0, slow_width=32)
    folder = write_random_model(raw, str(tmp_path / "positions"), seed=23, dtype=torch.bfloat16)
    sharpen_logits(folder)
    config, tensors = plain_model.read_model_folder(folder)
    assert tensors["model.position_table.weight"].shape == (320, 80)
    heads, kv_heads, width, eps = 3, 1, 64, config["rms_norm_eps"]
    half = 16
    frequency = 1.0 / np.power(np.float32(1e4), (2.0 * np.arange(half, dtype=np.float32)) / np.float32(32))
    angle = torch.from_numpy((np.arange(320, dtype=np.float32) / np.float32(4.0))[:, None] * frequency[None, :]).double()

    def turn(x, rotate):
        """x: [T, heads, 64], normalised already; rotates elements 0..31 in pairs (c, c + 16)."""
        if not rotate:
            return x
        n = x.shape[0]
        c, s = torch.cos(angle[:n])[:, None, :], torch.sin(angle[:n])[:, None, :]
        low, high = x[..., :half], x[..., half:2 * half]
        return torch.cat([low * c - high * s, high * c + low * s, x[..., 2 * half:]], dim=-1)

    def attention(rotate):
        def layer(x, prefix):
            w = lambda name: tensors[prefix + "self_attn." + name].double()
            n = x.shape[0]
            q = plain_model.rms_norm((x @ w("q_proj.weight").T).reshape(n, heads, width), w("q_norm.weight"), eps)
            k = plain_model.rms_norm((x @ w("k_proj.weight").T).reshape(n, kv_heads, width), w("k_norm.weight"), eps)
            v = (x @ w("v_proj.weight").T).reshape(n, kv_heads, width)
            return plain_model.causal_attention(turn(q, rotate), turn(k, rotate), v, None) @ w("o_proj.weight").T
        return layer

    def dense(x, prefix):
        return plain_model.gated_feed_forward(x, tensors, prefix + "mlp.")

    def add_positions(hidden):
        return hidden + tensors["model.position_table.weight"].double()[:hidden.shape[0]]

    requests = rh.random_requests(config["vocab_size"], [2, 64, 129, 257, 320], seed=24)
    expected = {name: plain_layers(config, tensors, tokens, [attention(False), attention(True)], [dense, dense], add_positions)
                for name, tokens in requests.items()}
    # The encodings matter: without the table, or with the usual rotation, the logits are others.
    bare = plain_layers(config, tensors, requests["r2"], [attention(False), attention(True)], [dense, dense])
    assert np.abs(bare - expected["r2"]).max() > 1e-2
    engine = Engine.load(folder, dtype=dtype, max_tokens=2048)
    run_every_way(engine, requests, expected, FP32_TOLERANCE if dtype == "float32" else BF16_TOLERANCE,
                  f"toy positions {dtype}")


# ------------------------------------------------- another norm and another arrangement
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_toy_norm_in_a_toy_arrangement(tmp_path, dtype):
    """A norm that subtracts the mean and has a bias, and a block that runs mixer and feed-forward
    side by side from one norm (out = x + mixer(n(x)) + feed_forward(n(x))), in the second of two
    layers; the first keeps the package's pre-norm block, whose last product must not prepare rows
    for a norm that it does not know. The final norm is the toy's too."""
    from kidi_b200 import Engine, register_architecture, register_part, write_random_model
    from kidi_b200.models import qwen3
    from kidi_b200.parts.base import Part, plain_rows
    from kidi_b200.parts.spec import LayerSpec, ParamSpec, PartSpec

    @register_part("norm", "toy_centred")
    class ToyCentredNorm(Part):
        def __init__(self, spec, env):
            super().__init__(spec, env)
            self.size, self.eps = int(spec.param("size")), float(spec.param("eps"))

        def parameter_specs(self):
            return [ParamSpec("weight", (self.size,), init=("one_plus_normal", 0.1)),
                    ParamSpec("bias", (self.size,), init=("normal", 0.1))]

        def bind(self, tensors):
            self.weight, self.bias = tensors["weight"].float(), tensors["bias"].float()

        def forward(self, stream, rows=None, scaled=False):
            delta = stream.take_pending()
            hidden = stream.hidden
            if rows is not None:                      # only these rows, the stream stays as it is
                hidden = hidden[rows.long()]
                if delta is not None:
                    hidden = hidden + delta[rows.long()].float()
            elif delta is not None:
                hidden += delta.float()
            centred = hidden - hidden.mean(dim=-1, keepdim=True)
            normed = centred * torch.rsqrt(centred.square().mean(dim=-1, keepdim=True) + self.eps)
            return (normed * self.weight + self.bias).to(self.env.dtype)

    @register_part("arrangement", "toy_side_by_side")
    class ToySideBySide(Part):
        ROLES = {"norm": "norm", "mixer": "mixer", "feed_forward": "feed_forward"}

        def __init__(self, spec, env, parts):
            super().__init__(spec, env)
            self.norm, self.mixer, self.feed_forward = parts["norm"], parts["mixer"], parts["feed_forward"]

        def children(self):
            return (self.norm, self.mixer, self.feed_forward)

        def cache_requests(self):
            return self.mixer.cache_requests()

        def first_norm(self):
            return self.norm

        def forward(self, stream, ctx, views, owns_cache):
            normed = plain_rows(self.norm.forward(stream))
            mixed = self.mixer.forward(normed, ctx, views, owns_cache)
            stream.add(mixed.float() + self.feed_forward.forward(normed, ctx).float())

    Config = wrapped_config(())

    def build(config):
        spec = qwen3.build_spec(config.base)
        centred = {"size": config.base.hidden_size, "eps": config.base.rms_norm_eps}
        second = spec.layers[1]
        side_by_side = LayerSpec(PartSpec("toy_side_by_side"), {
            "norm": PartSpec("toy_centred", centred, "model.layers.1.input_layernorm."),
            "mixer": second.parts["mixer"], "feed_forward": second.parts["feed_forward"]})
        return dataclasses.replace(spec, architecture="ToyNormForCausalLM", layers=(spec.layers[0], side_by_side),
                                   final_norm=PartSpec("toy_centred", centred, "model.norm."))

    register_architecture("ToyNormForCausalLM", Config, build)
    raw = dict(BASE, architectures=["ToyNormForCausalLM"])
    folder = write_random_model(raw, str(tmp_path / "norms"), seed=31, dtype=torch.bfloat16)
    sharpen_logits(folder)
    config, tensors = plain_model.read_model_folder(folder)
    assert "model.layers.1.post_attention_layernorm.weight" not in tensors and "model.norm.bias" in tensors
    eps = config["rms_norm_eps"]
    cos, sin = plain_model.rotary_tables(320, config["head_dim"], plain_model.rope_theta(config))

    def centred_norm(x, prefix):
        weight, bias = tensors[prefix + "weight"].double(), tensors[prefix + "bias"].double()
        centred = x - x.mean(dim=-1, keepdim=True)
        return centred * torch.rsqrt(centred.square().mean(dim=-1, keepdim=True) + eps) * weight + bias

    def whole(tokens):
        hidden = plain_model.embed(tokens, tensors["model.embed_tokens.weight"], torch.float64)
        n = len(tokens)
        hidden = plain_model.block(hidden, tensors, 0, config, cos[:n].double(), sin[:n].double(), None)
        normed = centred_norm(hidden, "model.layers.1.input_layernorm.")
        hidden = hidden + plain_model.attention_layer(normed, tensors, "model.layers.1.self_attn.", config,
                                                cos[:n].double(), sin[:n].double(), None) \
            + plain_model.gated_feed_forward(normed, tensors, "model.layers.1.mlp.")
        return (centred_norm(hidden, "model.norm.") @ tensors["lm_head.weight"].double().T).float().numpy()

    requests = rh.random_requests(config["vocab_size"], [2, 64, 129, 257, 320], seed=32)
    expected = {name: whole(tokens) for name, tokens in requests.items()}
    engine = Engine.load(folder, dtype=dtype, max_tokens=2048)
    run_every_way(engine, requests, expected, FP32_TOLERANCE if dtype == "float32" else BF16_TOLERANCE,
                  f"toy norm and arrangement {dtype}")


# ------------------------------------------------ scores that are bounded and shifted by position
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_with_bounded_and_shifted_scores(tmp_path, dtype):
    """The attention part's two options for its scores, set by a specification: layer 0 bounds them
    (cap * tanh(s / cap)), layer 1 shifts head h's by slope_h * (key position - query position).
    Nothing in the package's files changes; such layers run on the general attention kernel."""
    from kidi_b200 import Engine, register_architecture, write_random_model
    from kidi_b200.models import qwen3
    from kidi_b200.parts.spec import LayerSpec, PartSpec

    Config = wrapped_config(("cap", "slopes"))

    def build(config):
        spec = qwen3.build_spec(config.base)
        extras = ({"score_softcap": config.extra["cap"]}, {"score_slopes": config.extra["slopes"]})
        layers = []
        for layer, extra in zip(spec.layers, extras):
            parts = dict(layer.parts)
            mixer = parts["mixer"]
            parts["mixer"] = PartSpec(mixer.kind, dict(mixer.params, **extra), mixer.prefix)
            layers.append(LayerSpec(layer.arrangement, parts))
        return dataclasses.replace(spec, architecture="ToyScoresForCausalLM", layers=tuple(layers))

    register_architecture("ToyScoresForCausalLM", Config, build)
    cap, slopes = 1.5, [0.5, 0.125, 0.03125]
    raw = dict(BASE, architectures=["ToyScoresForCausalLM"], cap=cap, slopes=slopes)
    folder = write_random_model(raw, str(tmp_path / "scores"), seed=41, dtype=torch.bfloat16)
    sharpen_logits(folder)
    config, tensors = plain_model.read_model_folder(folder)
    heads, kv_heads, width, eps = 3, 1, 64, config["rms_norm_eps"]
    cos, sin = plain_model.rotary_tables(320, width, plain_model.rope_theta(config))

    def attention(reshape):
        def layer(x, prefix):
            w = lambda name: tensors[prefix + "self_attn." + name].double()
            n = x.shape[0]
            q = plain_model.norm_then_rotate((x @ w("q_proj.weight").T).reshape(n, heads, width), w("q_norm.weight"),
                                             eps, cos[:n].double(), sin[:n].double())
            k = plain_model.norm_then_rotate((x @ w("k_proj.weight").T).reshape(n, kv_heads, width), w("k_norm.weight"),
                                             eps, cos[:n].double(), sin[:n].double())
            v = (x @ w("v_proj.weight").T).reshape(n, kv_heads, width)
            out = torch.zeros(n, heads, width, dtype=torch.float64)
            distance = (torch.arange(n)[None, :] - torch.arange(n)[:, None]).double()       # key - query position
            hidden = distance > 0
            for head in range(heads):
                scores = reshape(q[:, head] @ k[:, 0].T / np.sqrt(width), head, distance)
                scores = scores.masked_fill(hidden, float("-inf"))
                out[:, head] = torch.softmax(scores, dim=-1) @ v[:, 0]
            return out.reshape(n, heads * width) @ w("o_proj.weight").T
        return layer

    bounded = attention(lambda s, head, distance: cap * torch.tanh(s / cap))
    shifted = attention(lambda s, head, distance: s + slopes[head] * distance)

    def dense(x, prefix):
        return plain_model.gated_feed_forward(x, tensors, prefix + "mlp.")

    requests = rh.random_requests(config["vocab_size"], [2, 64, 129, 257, 320], seed=42)
    expected = {name: plain_layers(config, tensors, tokens, [bounded, shifted], [dense, dense])
                for name, tokens in requests.items()}
    plain_scores = attention(lambda s, head, distance: s)
    usual = plain_layers(config, tensors, requests["r2"], [plain_scores, plain_scores], [dense, dense])
    assert np.abs(usual - expected["r2"]).max() > 1e-2        # the options matter
    engine = Engine.load(folder, dtype=dtype, max_tokens=2048)
    run_every_way(engine, requests, expected, FP32_TOLERANCE if dtype == "float32" else BF16_TOLERANCE,
                  f"bounded and shifted scores {dtype}")
