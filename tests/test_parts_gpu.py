"""Each part of a model alone against the plain implementation, and the generality of the assembly:
a toy mixer with state of its own, a toy architecture with different layers and a schedule that
runs a layer twice, all registered from here without touching the package."""

import tempfile
from dataclasses import dataclass

import numpy as np
import pytest
import torch

import helpers
import plain_gpt2

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def build_engine(which, dtype, **options):
    from pagedserve_b200.config.engine_config import EngineConfig
    from pagedserve_b200.engine.engine import Engine

    block = helpers.TINY[which][2]
    defaults = dict(dtype=dtype, block_size=block, num_blocks=1024 // block, max_num_seqs=8)
    defaults.update(options)
    return Engine.from_folder(helpers.model_folder(which), EngineConfig(**defaults))


def make_ctx(engine, entries):
    from pagedserve_b200.engine.batch import StepEntry

    ctx = engine.runner.prepare([StepEntry(*entry) for entry in entries])
    engine.runner.begin(ctx)          # the step's first kernel: positions, lengths and table rows from the slots
    return ctx


# ------------------------------------------------------------------ parts alone
@pytest.mark.parametrize("which", ["a", "b"])
@pytest.mark.parametrize("dtype,tol", [("float32", 2e-6), ("bfloat16", 6e-3)])
def test_each_part_alone(which, dtype, tol):
    """Embedding, norm, attention mixer, feed-forward and head of a real model, fed with the plain
    implementation's own intermediate values, one at a time."""
    engine = build_engine(which, dtype)
    config, weights = helpers.plain_model(which)
    hidden_size, heads, head_dim, _ = plain_gpt2.sizes(config)
    compute = engine.dtype
    tokens = helpers.random_tokens(config["vocab_size"], 45, seed=9)
    ids = torch.tensor(tokens)
    ctx = make_ctx(engine, [("x", tokens, [0, 44])])
    model = engine.model

    def close(got, want, limit=tol):
        want = want.double()
        error = float((got.double().cpu() - want).abs().max() / want.abs().max())
        assert error < limit, error

    # embedding + learned positions
    hidden = model.embedding.forward(ctx, model.positions)
    want_hidden = plain_gpt2.embedding(weights, ids, torch.arange(45))
    close(hidden, want_hidden, 1e-6)
    # norm
    block = model.blocks[1]
    eps = config["layer_norm_epsilon"]
    want_normed = plain_gpt2.layer_norm(want_hidden, weights["h.1.ln_1.weight"], weights["h.1.ln_1.bias"], eps)
    normed = block.norms["pre_mixer"].forward(want_hidden.float().to(DEV))
    close(normed, want_normed)
    # attention mixer (writes the cache of layer 1, reads it back)
    from pagedserve_b200.parts.base import LayerContext

    layer = LayerContext(1, 1, model.positions)
    group = engine.cache.groups[0]
    layer.k_pool, layer.v_pool = group.layer_views(1)
    layer.page_stride, layer.page_size, layer.block_table = group.page_stride, group.page_size, ctx.block_tables[0]
    residual = torch.zeros(45, hidden_size, dtype=torch.float32, device=DEV)
    block.mixer.forward(want_normed.to(compute).to(DEV), residual, ctx, layer)
    close(residual, plain_gpt2.attention_sublayer(weights, "h.1.", want_normed, heads, head_dim), max(tol, 1e-5))
    # feed-forward
    residual.zero_()
    block.feed_forward.forward(want_normed.to(compute).to(DEV), residual, ctx)
    close(residual, plain_gpt2.mlp_sublayer(weights, "h.1.", want_normed, config["activation_function"]),
          max(tol, 1e-5))
    # final norm on the wanted rows + head
    picked = model.final_norm.forward(want_hidden.float().to(DEV), rows=ctx.logit_rows)
    logits = model.head.forward(picked, model.embedding)
    close(logits, plain_gpt2.lm_head(weights, config, want_hidden)[[0, 44]], max(tol, 1e-5))
    # whole block (pre-norm arrangement) in place on the float32 stream
    stream = want_hidden.float().to(DEV).clone()
    block.forward(stream, ctx, layer)
    close(stream, plain_gpt2.block(weights, 1, want_hidden, config), max(tol, 1e-5))
    engine.cache.rollback("x")
    engine.cache.free("x")


# ------------------------------------------------------------------ a toy mixer with state, a toy architecture
def register_toy():
    """A decayed running sum over the tokens of a request: y_t = s_t W, s_t = decay * s_{t-1} + x_t.
    The sum ``s`` is per-request state of fixed size kept in the request's slot."""
    from pagedserve_b200.cache.manager import StateNeed
    from pagedserve_b200.config.registry import ModelConfig, register_architecture
    from pagedserve_b200.models.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
    from pagedserve_b200.parts.base import Mixer, register_part
    from pagedserve_b200.weights.loader import ParamSpec

    @register_part("mixer", "toy_running_sum", replace=True)
    class RunningSum(Mixer):
        def state_need(self):
            return StateNeed((self.params["width"],), "float32")

        def param_specs(self):
            width = self.params["width"]
            return [(ParamSpec(self._n("mix.weight"), (width, width), "matmul"), ("normal", 0.05))]

        def bind(self, tensors):
            self.weight = tensors[self._n("mix.weight")]

        def forward(self, x, residual, ctx, layer):
            decay = self.params["decay"]
            host = ctx.host
            for item in range(ctx.num_items):                      # a request's tokens run in order
                slot = int(host.item_slot[item])
                begin, end = int(host.q_start[item]), int(host.q_start[item + 1])
                state = layer.state[slot]
                outputs = []
                for token in range(begin, end):
                    state.mul_(decay).add_(x[token].float())
                    outputs.append(state.clone())
                mixed = torch.stack(outputs).to(self.env.dtype)
                out = torch.empty(end - begin, self.weight.shape[0], dtype=torch.float32, device=x.device)
                self.env.ops.linear(mixed, self.weight, None, out)
                residual[begin:end] += out

    @dataclass
    class ToyConfig(ModelConfig):
        width: int = 32
        vocab: int = 97
        max_len: int = 64
        decay: float = 0.5

        @classmethod
        def from_dict(cls, values):
            return cls(values["width"], values["vocab"], values["max_len"], values["decay"])

        def to_dict(self):
            return {"architectures": ["ToyMixedLM"], "width": self.width, "vocab": self.vocab,
                    "max_len": self.max_len, "decay": self.decay}

        architecture = property(lambda self: "ToyMixedLM")
        vocabulary_size = property(lambda self: self.vocab)
        max_model_len = property(lambda self: self.max_len)

    def build(config):
        width = config.width
        norm = dict(width=width, eps=1e-5, has_mean=False, has_bias=False, init_std=0.02)     # RMS form
        mlp = PartSpec("dense_mlp", dict(hidden_size=width, inner_size=48, activation="gelu_erf", has_bias=False,
                                         stored_in_out=False, up_name="up", down_name="down"), "")

        def layer(index, mixer):
            prefix = f"layers.{index}."
            return LayerSpec(PartSpec("pre_norm"), PartSpec(mixer.kind, mixer.params, prefix),
                             PartSpec(mlp.kind, mlp.params, prefix),
                             {"pre_mixer": PartSpec("layernorm", dict(norm, name="n1"), prefix),
                              "pre_feed_forward": PartSpec("layernorm", dict(norm, name="n2"), prefix)})

        toy = PartSpec("toy_running_sum", dict(width=width, decay=config.decay))
        attention = PartSpec("causal_attention", dict(hidden_size=width, n_heads=2, n_kv_heads=1, head_dim=16,
                                                      scale=0.25, window=9, has_bias=False, stored_in_out=False,
                                                      qkv_name="qkv", out_name="o"))
        return ModelSpec(
            architecture="ToyMixedLM", hidden_size=width, vocab_size=config.vocab, max_model_len=config.max_len,
            embedding=PartSpec("token_embedding", dict(vocab_size=config.vocab, hidden_size=width, name="emb")),
            positions=PartSpec("none"),
            layers=[layer(0, toy), layer(1, attention)],
            # different mixers in different layers; the attention layer runs twice, each run on a
            # cache layer of its own
            schedule=[ScheduleEntry(0, 0), ScheduleEntry(1, 1), ScheduleEntry(1, 2)],
            final_norm=PartSpec("layernorm", dict(norm, name="norm_f")),
            head=PartSpec("lm_head", dict(vocab_size=config.vocab, hidden_size=width, tied=True, name="head")))

    register_architecture("ToyMixedLM", ToyConfig, build, replace=True)
    return ToyConfig


def toy_plain(tensors, config, tokens):
    """The toy model, whole sequence, no cache, float64."""
    w = {name: t.double() for name, t in tensors.items()}

    def rms(x, gain):
        return x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-5) * gain

    def mlp(x, prefix):
        return plain_gpt2.activation(x @ w[prefix + "up.weight"].T, "gelu") @ w[prefix + "down.weight"].T

    h = w["emb.weight"][torch.tensor(tokens)]
    x = rms(h, w["layers.0.n1.weight"])
    state = torch.zeros(config.width, dtype=torch.float64)
    sums = []
    for row in x:
        state = config.decay * state + row
        sums.append(state)
    h = h + torch.stack(sums) @ w["layers.0.mix.weight"].T
    h = h + mlp(rms(h, w["layers.0.n2.weight"]), "layers.0.")
    for _ in range(2):
        x = rms(h, w["layers.1.n1.weight"])
        qkv = x @ w["layers.1.qkv.weight"].T
        q = qkv[:, :32].reshape(-1, 2, 16)
        k = qkv[:, 32:48].reshape(-1, 1, 16).repeat_interleave(2, 1)
        v = qkv[:, 48:].reshape(-1, 1, 16).repeat_interleave(2, 1)
        # plain_gpt2.causal_attention scales by head_dim^-0.5 = 0.25, the toy's scale
        h = h + plain_gpt2.causal_attention(q, k, v, window=9) @ w["layers.1.o.weight"].T
        h = h + mlp(rms(h, w["layers.1.n2.weight"]), "layers.1.")
    return rms(h, w["norm_f.weight"]) @ w["emb.weight"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_mixer_with_state_registers_builds_and_steps(dtype):
    from pagedserve_b200.config.engine_config import EngineConfig
    from pagedserve_b200.engine.batch import StepEntry
    from pagedserve_b200.engine.engine import Engine
    from pagedserve_b200.weights.random_init import write_random_model
    from pagedserve_b200.weights.safetensors_io import read_safetensors

    ToyConfig = register_toy()
    config = ToyConfig()
    with tempfile.TemporaryDirectory() as folder:
        write_random_model(folder, config, seed=3)
        tensors = read_safetensors(folder + "/model.safetensors")
        engine = Engine.from_folder(folder, EngineConfig(dtype=dtype, block_size=4, num_blocks=16, max_num_seqs=3))
    assert len(engine.cache.groups) == 1 and engine.cache.groups[0].need.window == 9
    assert list(engine.cache.state) == [0]                       # the toy mixer's slot state
    sequences = {"a": helpers.random_tokens(97, 40, seed=1), "b": helpers.random_tokens(97, 23, seed=2)}
    want = {name: toy_plain(tensors, config, tokens).numpy() for name, tokens in sequences.items()}
    # portions of a beside portions and single tokens of b; the window lets pages go while a request lives
    plan = [[("a", 0, 7), ("b", 0, 1)], [("a", 7, 9), ("b", 1, 6)], [("b", 6, 7)], [("a", 9, 30), ("b", 7, 23)],
            [("a", 30, 31)], [("a", 31, 40)]]
    got = {"a": [], "b": []}
    for step in plan:
        entries = [StepEntry(name, sequences[name][lo:hi], list(range(hi - lo))) for name, lo, hi in step]
        logits = engine.step(entries).cpu().numpy()
        cursor = 0
        for name, lo, hi in step:
            got[name].append(logits[cursor:cursor + hi - lo])
            cursor += hi - lo
    assert engine.cache.groups[0].allocator.used_pages <= 8       # 63 tokens would need 16 pages of 4: the window gave pages back
    for name in sequences:
        helpers.assert_close(np.concatenate(got[name]), want[name], dtype, f"toy/{name}")
    # a slot that is handed out again starts from zero state
    engine.finish("a")
    engine.finish("b")
    again = engine.step([StepEntry("c", sequences["b"], list(range(23)))]).cpu().numpy()
    helpers.assert_close(again, want["b"], dtype, "toy/slot reuse")
    engine.cache.check_invariants()


# ----------------------------------------------------------------------------------------------
# Another position encoding and a feed-forward with routing, both defined here: the interfaces of
# pagedserve_b200.parts are enough to register, build and step them.
# ----------------------------------------------------------------------------------------------
def register_rotary_routed_toy():
    from pagedserve_b200.config.registry import ModelConfig, register_architecture
    from pagedserve_b200.models.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
    from pagedserve_b200.parts.base import FeedForward, PositionEncoding, register_part
    from pagedserve_b200.weights.loader import ParamSpec

    @register_part("positions", "toy_rotary", replace=True)
    class ToyRotary(PositionEncoding):
        """Pairs (i, i + head_dim / 2) of every head of q and k turn by position * base^(-2i / head_dim),
        angles and products in float32; the keys go into the cache already turned."""

        def rotate(self, q, k, ctx):
            head_dim, base = self.params["head_dim"], self.params["base"]
            half = head_dim // 2
            inv = base ** (-torch.arange(half, dtype=torch.float32, device=q.device) * 2.0 / head_dim)
            angle = ctx.positions.to(torch.float32)[:, None] * inv[None, :]            # [T, half]
            cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
            for tensor in (q, k):
                heads = tensor.shape[1] // head_dim
                x = tensor.reshape(tensor.shape[0], heads, head_dim).to(torch.float32)
                lo, hi = x[..., :half], x[..., half:]
                turned = torch.cat([lo * cos - hi * sin, hi * cos + lo * sin], dim=-1)
                tensor.copy_(turned.reshape(tensor.shape[0], heads * head_dim).to(tensor.dtype))

    @register_part("feed_forward", "toy_top1_experts", replace=True)
    class TopOneExperts(FeedForward):
        """Router logits in float32; every token goes to its best expert, whose output is scaled by the
        softmax weight of that expert. The grouping of tokens by expert is host logic."""

        def param_specs(self):
            p = self.params
            E, H, I = p["n_experts"], p["hidden_size"], p["inner_size"]
            return [(ParamSpec(self._n("router.weight"), (E, H), "keep32"), ("normal", 0.5)),
                    (ParamSpec(self._n("experts.up"), (E, I, H), "matmul"), ("normal", 0.05)),
                    (ParamSpec(self._n("experts.down"), (E, H, I), "matmul"), ("normal", 0.05))]

        def bind(self, tensors):
            self.router = tensors[self._n("router.weight")]
            self.up = tensors[self._n("experts.up")]
            self.down = tensors[self._n("experts.down")]

        def forward(self, x, residual, ctx):
            ops = self.env.ops
            weights = torch.softmax(x.to(torch.float32) @ self.router.to(torch.float32).T, dim=-1)
            gate, choice = weights.max(dim=-1)
            for expert in range(self.params["n_experts"]):
                rows = torch.nonzero(choice == expert).reshape(-1)                      # host sync: which tokens
                if rows.numel() == 0:
                    continue
                picked = x[rows].contiguous()
                inner = torch.empty(rows.numel(), self.up.shape[1], dtype=self.env.dtype, device=x.device)
                ops.linear(picked, self.up[expert], None, inner, act="gelu_tanh")
                out = torch.empty(rows.numel(), self.down.shape[1], dtype=torch.float32, device=x.device)
                ops.linear(inner, self.down[expert], None, out)
                residual.index_add_(0, rows, out * gate[rows, None])

    @dataclass
    class ToyConfig(ModelConfig):
        width: int = 64
        vocab: int = 131
        max_len: int = 96
        n_experts: int = 3

        @classmethod
        def from_dict(cls, values):
            return cls(values["width"], values["vocab"], values["max_len"], values["n_experts"])

        def to_dict(self):
            return {"architectures": ["ToyRotaryRoutedLM"], "width": self.width, "vocab": self.vocab,
                    "max_len": self.max_len, "n_experts": self.n_experts}

        architecture = property(lambda self: "ToyRotaryRoutedLM")
        vocabulary_size = property(lambda self: self.vocab)
        max_model_len = property(lambda self: self.max_len)

    def build(config):
        width = config.width
        norm = dict(width=width, eps=1e-6, has_mean=True, has_bias=True, init_std=0.02)

        def layer(index):
            prefix = f"blocks.{index}."
            mixer = PartSpec("causal_attention", dict(hidden_size=width, n_heads=2, n_kv_heads=2, head_dim=32,
                                                      scale=32 ** -0.5, window=None, has_bias=True,
                                                      stored_in_out=False, qkv_name="qkv", out_name="o"), prefix)
            experts = PartSpec("toy_top1_experts", dict(hidden_size=width, inner_size=80,
                                                        n_experts=config.n_experts), prefix)
            return LayerSpec(PartSpec("pre_norm"), mixer, experts,
                             {"pre_mixer": PartSpec("layernorm", dict(norm, name="n1"), prefix),
                              "pre_feed_forward": PartSpec("layernorm", dict(norm, name="n2"), prefix)})

        return ModelSpec(
            architecture="ToyRotaryRoutedLM", hidden_size=width, vocab_size=config.vocab,
            max_model_len=config.max_len,
            embedding=PartSpec("token_embedding", dict(vocab_size=config.vocab, hidden_size=width, name="emb")),
            positions=PartSpec("toy_rotary", dict(head_dim=32, base=100.0)),
            layers=[layer(0), layer(1)], schedule=[ScheduleEntry(0, 0), ScheduleEntry(1, 1)],
            final_norm=PartSpec("layernorm", dict(norm, name="norm_f")),
            head=PartSpec("lm_head", dict(vocab_size=config.vocab, hidden_size=width, tied=True, name="head")))

    register_architecture("ToyRotaryRoutedLM", ToyConfig, build, replace=True)
    return ToyConfig


def rotary_routed_plain(tensors, config, tokens):
    """The same model, whole sequence, no cache, float64."""
    w = {name: t.double() for name, t in tensors.items()}
    T = len(tokens)

    def norm(x, prefix):
        return plain_gpt2.layer_norm(x, w[prefix + ".weight"], w[prefix + ".bias"], 1e-6)

    def turn(x):                                   # [T, heads, 32]
        half = 16
        inv = 100.0 ** (-torch.arange(half, dtype=torch.float64) * 2.0 / 32)
        angle = torch.arange(T, dtype=torch.float64)[:, None] * inv[None, :]
        cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
        lo, hi = x[..., :half], x[..., half:]
        return torch.cat([lo * cos - hi * sin, hi * cos + lo * sin], dim=-1)

    h = w["emb.weight"][torch.tensor(tokens)]
    for index in range(2):
        p = f"blocks.{index}."
        qkv = norm(h, p + "n1") @ w[p + "qkv.weight"].T + w[p + "qkv.bias"]
        q, k, v = (qkv[:, i * 64:(i + 1) * 64].reshape(T, 2, 32) for i in range(3))
        h = h + plain_gpt2.causal_attention(turn(q), turn(k), v).reshape(T, 64) @ w[p + "o.weight"].T + w[p + "o.bias"]
        x = norm(h, p + "n2")
        weights = torch.softmax(x @ w[p + "router.weight"].T, dim=-1)
        gate, choice = weights.max(dim=-1)
        out = torch.zeros_like(h)
        for t in range(T):
            e = int(choice[t])
            inner = plain_gpt2.activation(x[t] @ w[p + "experts.up"][e].T, "gelu_new")
            out[t] = gate[t] * (inner @ w[p + "experts.down"][e].T)
        h = h + out
    return norm(h, "norm_f") @ w["emb.weight"].T


@pytest.mark.parametrize("dtype,n_experts", [("float32", 3), ("bfloat16", 1)])
def test_toy_position_encoding_and_routed_feed_forward(dtype, n_experts):
    """A rotary position encoding and a routed feed-forward that exist only in this test run through the
    framework's registry, loader, cache and step function: whole prompts, portions and single tokens give
    the logits of a plain implementation. (In bfloat16 with several experts a near-tie of the router may fall
    the other way than in float64, which says nothing about the framework: that case runs one expert.)"""
    from pagedserve_b200.config.engine_config import EngineConfig
    from pagedserve_b200.engine.batch import StepEntry
    from pagedserve_b200.engine.engine import Engine
    from pagedserve_b200.weights.random_init import write_random_model
    from pagedserve_b200.weights.safetensors_io import read_safetensors

    ToyConfig = register_rotary_routed_toy()
    config = ToyConfig(n_experts=n_experts)
    with tempfile.TemporaryDirectory() as folder:
        write_random_model(folder, config, seed=7)
        tensors = read_safetensors(folder + "/model.safetensors")
        engine = Engine.from_folder(folder, EngineConfig(dtype=dtype, block_size=8, num_blocks=24, max_num_seqs=3))
    assert not engine.runner.enable_cuda_graphs          # parts with host logic run eagerly
    sequences = {"a": helpers.random_tokens(131, 50, seed=4), "b": helpers.random_tokens(131, 31, seed=5)}
    want = {name: rotary_routed_plain(tensors, config, tokens).numpy() for name, tokens in sequences.items()}
    plan = [[("a", 0, 20)], [("a", 20, 21), ("b", 0, 17)], [("a", 21, 22), ("b", 17, 19)], [("a", 22, 49), ("b", 19, 20)],
            [("a", 49, 50), ("b", 20, 31)]]
    got = {"a": [], "b": []}
    for step in plan:
        entries = [StepEntry(name, sequences[name][lo:hi], list(range(hi - lo))) for name, lo, hi in step]
        logits = engine.step(entries).cpu().numpy()
        cursor = 0
        for name, lo, hi in step:
            got[name].append(logits[cursor:cursor + hi - lo])
            cursor += hi - lo
    for name in sequences:
        helpers.assert_close(np.concatenate(got[name]), want[name], dtype, f"rotary+routed/{name}")
    engine.finish("a")
    engine.finish("b")
    engine.cache.check_invariants()


# ----------------------------------------------------------------------------------------------
# A mixer with state of its own that runs on the device alone (its steps are captured as CUDA graphs):
# the runner must not launch a step ahead of its tokens for such a model, because a step that is launched
# and then dropped (a request ended on an end-of-sequence token) would have moved the slots' state on.
# ----------------------------------------------------------------------------------------------
def register_device_state_toy():
    from pagedserve_b200.cache.manager import StateNeed
    from pagedserve_b200.config.registry import ModelConfig, register_architecture
    from pagedserve_b200.models.spec import LayerSpec, ModelSpec, PartSpec
    from pagedserve_b200.parts.base import Mixer, register_part
    from pagedserve_b200.weights.loader import ParamSpec

    @register_part("mixer", "toy_device_running_sum", replace=True)
    class DeviceRunningSum(Mixer):
        """y_t = s_t W with s_t = decay * s_{t-1} + x_t per request, s kept in the request's slot; computed
        from the step's device arrays only (no host logic), so the step can be a CUDA graph."""

        graph_safe = True

        def state_need(self):
            return StateNeed((self.params["width"],), "float32")

        def param_specs(self):
            width = self.params["width"]
            return [(ParamSpec(self._n("mix.weight"), (width, width), "matmul"), ("normal", 0.05))]

        def bind(self, tensors):
            self.weight = tensors[self._n("mix.weight")]

        def forward(self, x, residual, ctx, layer):
            decay = self.params["decay"]
            tokens = x.shape[0]
            item, slot = ctx.token_item.long(), ctx.token_slot.long()
            index = torch.arange(tokens, device=x.device)
            first = ctx.q_start.long()[item]                                  # first token of each token's entry
            gap = (index[:, None] - index[None, :]).clamp(min=0).to(torch.float32)
            weights = torch.where((item[:, None] == item[None, :]) & (index[None, :] <= index[:, None]),
                                  decay ** gap, torch.zeros_like(gap))
            carried = (decay ** (index - first + 1).to(torch.float32))[:, None] * layer.state[slot]
            sums = weights @ x.to(torch.float32) + carried                    # the state after every token
            last = (ctx.q_start.long()[1:] - 1).clamp(min=0)                  # last token of every entry
            layer.state[ctx.item_slot.long()] = sums[last]
            self.env.ops.linear(sums.to(self.env.dtype), self.weight, None, residual, accumulate=True)

    @dataclass
    class StateToyConfig(ModelConfig):
        width: int = 32
        vocab: int = 61
        max_len: int = 48
        decay: float = 0.6

        @classmethod
        def from_dict(cls, values):
            return cls(values["width"], values["vocab"], values["max_len"], values["decay"])

        def to_dict(self):
            return {"architectures": ["ToyDeviceStateLM"], "width": self.width, "vocab": self.vocab,
                    "max_len": self.max_len, "decay": self.decay}

        architecture = property(lambda self: "ToyDeviceStateLM")
        vocabulary_size = property(lambda self: self.vocab)
        max_model_len = property(lambda self: self.max_len)

    def build(config):
        width = config.width
        norm = dict(width=width, eps=1e-5, has_mean=False, has_bias=False, init_std=0.02)
        layer = LayerSpec(
            PartSpec("pre_norm"), PartSpec("toy_device_running_sum", dict(width=width, decay=config.decay), "l0."),
            PartSpec("dense_mlp", dict(hidden_size=width, inner_size=40, activation="gelu_tanh", has_bias=False,
                                       stored_in_out=False, up_name="up", down_name="down"), "l0."),
            {"pre_mixer": PartSpec("layernorm", dict(norm, name="n1"), "l0."),
             "pre_feed_forward": PartSpec("layernorm", dict(norm, name="n2"), "l0.")})
        return ModelSpec(
            architecture="ToyDeviceStateLM", hidden_size=width, vocab_size=config.vocab,
            max_model_len=config.max_len,
            embedding=PartSpec("token_embedding", dict(vocab_size=config.vocab, hidden_size=width, name="emb")),
            positions=PartSpec("none"), layers=[layer], schedule=[],
            final_norm=PartSpec("layernorm", dict(norm, name="norm_f")),
            head=PartSpec("lm_head", dict(vocab_size=config.vocab, hidden_size=width, tied=True, name="head")))

    register_architecture("ToyDeviceStateLM", StateToyConfig, build, replace=True)
    return StateToyConfig


def device_state_toy_generate(tensors, config, prompt, count):
    """Greedy tokens of the toy model above, whole sequence each time, float64."""
    w = {name: t.double() for name, t in tensors.items()}
    rms = lambda x, gain: x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-5) * gain
    tokens, produced = list(prompt), []
    for _ in range(count):
        h = w["emb.weight"][torch.tensor(tokens)]
        state, sums = torch.zeros(config.width, dtype=torch.float64), []
        for row in rms(h, w["l0.n1.weight"]):
            state = config.decay * state + row
            sums.append(state)
        h = h + torch.stack(sums) @ w["l0.mix.weight"].T
        inner = plain_gpt2.activation(rms(h, w["l0.n2.weight"]) @ w["l0.up.weight"].T, "gelu_new")
        h = h + inner @ w["l0.down.weight"].T
        logits = rms(h[-1], w["norm_f.weight"]) @ w["emb.weight"].T
        tokens.append(int(torch.argmax(logits)))
        produced.append(tokens[-1])
    return produced


def test_graph_safe_mixer_with_slot_state_survives_a_request_that_ends_early():
    from pagedserve_b200.config.engine_config import EngineConfig
    from pagedserve_b200.engine.engine import Engine
    from pagedserve_b200.weights.random_init import write_random_model
    from pagedserve_b200.weights.safetensors_io import read_safetensors

    StateToyConfig = register_device_state_toy()
    config = StateToyConfig()
    with tempfile.TemporaryDirectory() as folder:
        write_random_model(folder, config, seed=11)
        tensors = read_safetensors(folder + "/model.safetensors")
        engine = Engine.from_folder(folder, EngineConfig(dtype="float32", block_size=4, num_blocks=8, max_num_seqs=4))
    assert engine.model.graph_safe and engine.runner.enable_cuda_graphs
    assert list(engine.cache.state) == [0] and not engine.cache.groups     # slot state only, no pages at all
    prompts = [helpers.random_tokens(config.vocab, n, seed=60 + n) for n in (5, 9, 12)]
    want = [device_state_toy_generate(tensors, config, prompt, 14) for prompt in prompts]
    eos = want[1][4]                                                   # request 1 ends on its fifth token
    for produced in want:
        if eos in produced:
            del produced[produced.index(eos) + 1:]
    assert len(want[1]) == 5 and max(len(produced) for produced in want) > 8
    scheduler = engine.make_scheduler(strategy="orca", max_num_seqs=4, eos_token_id=eos)
    ids = [scheduler.add_token_request(prompt, max_new_tokens=14) for prompt in prompts]
    while scheduler.waiting or scheduler.active:
        scheduler.step()
        staged = engine.runner._staged
        assert staged is None or not staged.launched                    # prepared ahead at most, never launched
    assert engine.runner.graph_replays > 0                              # the decode steps did run as graphs
    assert [scheduler.finished[i].generated_token_ids for i in ids] == want
    engine.check_status()
