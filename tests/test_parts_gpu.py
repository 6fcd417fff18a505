"""Each part alone against its plain function, a model whose order runs a layer twice and
shares a cache, and toy parts defined here — a mixer with state of its own, a feed-forward
with routing, a rotary position encoding — that are registered, built and stepped without
touching the package's files."""

from __future__ import annotations

import dataclasses
import math

import pytest
import torch

import plain_gpt2 as plain
from ayaka_b200.engine.core import EngineCore
from ayaka_b200.engine.runner import StepEntry
from ayaka_b200.models.decoder import DecoderModel
from ayaka_b200.parts import (BuildContext, LayerSpec, ModelSpec, PartSpec, Run, StateNeed,
                              build_part, register_part)
from ayaka_b200.parts.embedding import PositionEncoding
from ayaka_b200.parts.feed_forward import FeedForward
from ayaka_b200.parts.mixer import Mixer

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def fill(part, seed=0, scale=0.3):
    """Random parameters; norm scales around 1. Returns {name: float32 cpu copy}."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, param in part.named_params():
        value = torch.randn(param.tensor.shape, generator=g) * scale
        if name.endswith("norm.weight"):
            value += 1.0
        param.tensor.copy_(value.to(param.tensor.dtype))
        out[name] = param.tensor.float().cpu()
    return out


def model_spec(layers, order, width, vocab=61, positions=96, position_kind="learned"):
    norm = PartSpec("layer_norm", width=width, eps=1e-5, bias=True)
    if isinstance(position_kind, PartSpec):
        position = position_kind
    else:
        position = PartSpec("learned", max_positions=positions, width=width) \
            if position_kind == "learned" else PartSpec("none")
    return ModelSpec(hidden_size=width, vocab_size=vocab, max_positions=positions,
                     embedding=PartSpec("token", vocab_size=vocab, width=width),
                     position=position, layers=tuple(layers), order=tuple(order),
                     final_norm=norm, head=PartSpec("linear", vocab_size=vocab, width=width,
                                                    tied=True))


def attention_layer(width, heads, kv_heads, head_dim, scale, inner, act="gelu_tanh", window=0):
    norm = PartSpec("layer_norm", width=width, eps=1e-5, bias=True)
    return LayerSpec("pre_norm",
                     PartSpec("attention", width=width, num_heads=heads, num_kv_heads=kv_heads,
                              head_dim=head_dim, scale=scale, window=window, bias=True),
                     PartSpec("dense", width=width, inner=inner, activation=act, bias=True),
                     norm, norm)


def core_of(spec, dtype="float32", pages=40, page=8, running=3, rows=128):
    ctx = BuildContext(torch.float32 if dtype == "float32" else torch.bfloat16, DEV)
    model = DecoderModel(spec, ctx)
    weights = fill(model)
    core = EngineCore(model, None, dtype=dtype, device=DEV, block_size=page, num_blocks=pages,
                      max_running=running, max_tokens_per_step=rows, poison_cache=True)
    return core, weights


def feed(core, rid, tokens, cuts):
    """Feed ``tokens`` in portions of the given sizes; logits at every position."""
    out, at = [], 0
    for size in cuts:
        part = tokens[at:at + size]
        out.append(core.step([StepEntry(rid, part, list(range(len(part))))]).cpu())
        at += len(part)
    assert at == len(tokens)
    return torch.cat(out)


# ---- plain versions of generic blocks ---------------------------------------------------------
def plain_attention_layer(x, w, prefix, heads, kv_heads, head_dim, scale, act, window=0,
                          kv_from=None):
    """One pre-norm layer with grouped-query attention from parameters named as the parts
    name them ([out, in] matrices). ``kv_from``: (k, v) of another run to attend over."""
    steps = x.shape[0]
    h = plain.layer_norm(x, w[prefix + "mixer_norm.weight"], w[prefix + "mixer_norm.bias"], 1e-5)
    qkv = h @ w[prefix + "mixer.qkv.weight"].t() + w[prefix + "mixer.qkv.bias"]
    q, k, v = qkv.split([heads * head_dim, kv_heads * head_dim, kv_heads * head_dim], dim=-1)
    q = q.reshape(steps, heads, head_dim)
    k = k.reshape(steps, kv_heads, head_dim)
    v = v.reshape(steps, kv_heads, head_dim)
    if kv_from is not None:
        k, v = kv_from
    rep = heads // kv_heads
    attended = plain.causal_attention(q, k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1),
                                      scale, window).reshape(steps, heads * head_dim)
    x = x + attended @ w[prefix + "mixer.out.weight"].t() + w[prefix + "mixer.out.bias"]
    h = plain.layer_norm(x, w[prefix + "feed_forward_norm.weight"],
                         w[prefix + "feed_forward_norm.bias"], 1e-5)
    name = "gelu_new" if act == "gelu_tanh" else "gelu"
    inner = plain.gelu(h @ w[prefix + "feed_forward.up.weight"].t()
                       + w[prefix + "feed_forward.up.bias"], name)
    x = x + inner @ w[prefix + "feed_forward.down.weight"].t() + w[prefix + "feed_forward.down.bias"]
    return x, (k, v)


def plain_head(x, w):
    h = plain.layer_norm(x, w["final_norm.weight"], w["final_norm.bias"], 1e-5)
    return h @ w["embedding.weight"].t()


# ---- parts alone ------------------------------------------------------------------------------
def test_norm_part_alone():
    ctx = BuildContext(torch.float32, DEV)
    norm = build_part("norm", "layer_norm", PartSpec("layer_norm", width=100, eps=1e-3, bias=True),
                      ctx)
    w = fill(norm, 1)
    x = torch.randn(7, 100, device=DEV) * 4
    out = torch.zeros(7, 100, device=DEV)
    norm.forward(x, out, count=7)
    torch.testing.assert_close(out.cpu(), plain.layer_norm(x.cpu(), w["weight"], w["bias"], 1e-3),
                               rtol=1e-5, atol=1e-5)
    nobias = build_part("norm", "layer_norm", PartSpec("layer_norm", width=100, eps=1e-3,
                                                       bias=False), ctx)
    assert [name for name, _ in nobias.named_params()] == ["weight"]


def test_feed_forward_part_alone():
    from ayaka_b200.parts.context import StepContext, Workspace

    ctx = BuildContext(torch.float32, DEV)
    for act in ("gelu_tanh", "gelu_erf"):
        mlp = build_part("feed_forward", "dense",
                         PartSpec("dense", width=40, inner=104, activation=act, bias=True), ctx)
        w = fill(mlp, 2)
        h = torch.randn(9, 40, device=DEV)
        residual = torch.randn(9, 40, device=DEV)
        before = residual.cpu().clone()
        empty = torch.zeros(1, dtype=torch.int32, device=DEV)
        step = StepContext(9, 1, empty, empty, empty, empty, empty, empty, [9], [0], [0], [],
                           Workspace(16, DEV), empty)
        mlp.forward(h, residual, step)
        name = "gelu_new" if act == "gelu_tanh" else "gelu"
        inner = plain.gelu(h.cpu() @ w["up.weight"].t() + w["up.bias"], name)
        expected = before + inner @ w["down.weight"].t() + w["down.bias"]
        torch.testing.assert_close(residual.cpu(), expected, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("dtype,tol", [("float32", 1e-4), ("bfloat16", 4e-2)])
def test_attention_and_block_parts_in_a_one_layer_model(dtype, tol):
    """Grouped-query heads (6 over 2), head size 48, a window of 20, erf GELU: options GPT-2
    never uses, given to the parts as parameters."""
    layer = attention_layer(96, 6, 2, 16, 0.3, 200, act="gelu_erf", window=20)
    core, w = core_of(model_spec([layer], [Run(0)], 96), dtype)
    tokens = [(7 * i + 3) % 61 for i in range(70)]
    got = feed(core, "a", tokens, (33, 2, 1, 1, 30, 3))
    x = w["embedding.weight"][tokens] + w["position.weight"][:70]
    x, _ = plain_attention_layer(x, w, "layers.0.", 6, 2, 16, 0.3, "gelu_erf", window=20)
    expected = plain_head(x, w)
    scale = float(expected.abs().max())
    assert float((got - expected).abs().max()) <= tol * scale
    # the windowed group gave pages back while the request was still running
    assert core.manager.num_free_pages() > core.manager.pools[0].num_usable - 9
    core.release("a")
    core.manager.check_integrity()


def test_order_runs_a_layer_twice_and_shares_a_cache():
    """Order: layer 0, layer 1, layer 0 again (own cache slot), layer 2 reading run 1's cache."""
    layers = [attention_layer(64, 4, 4, 16, 0.25, 96), attention_layer(64, 4, 2, 16, 0.2, 80),
              attention_layer(64, 4, 2, 16, 0.35, 72, act="gelu_erf")]
    order = [Run(0), Run(1), Run(0), Run(2, reads_cache_of=1)]
    core, w = core_of(model_spec(layers, order, 64))
    assert core.cache_plan.slots_per_group == (2, 1) and len(core.cache_plan.groups) == 2
    tokens = [(5 * i + 1) % 61 for i in range(50)]
    got = feed(core, "a", tokens, (20, 7, 1, 1, 21))
    x = w["embedding.weight"][tokens] + w["position.weight"][:50]
    x, _ = plain_attention_layer(x, w, "layers.0.", 4, 4, 16, 0.25, "gelu_tanh")
    x, kv1 = plain_attention_layer(x, w, "layers.1.", 4, 2, 16, 0.2, "gelu_tanh")
    x, _ = plain_attention_layer(x, w, "layers.0.", 4, 4, 16, 0.25, "gelu_tanh")
    x, _ = plain_attention_layer(x, w, "layers.2.", 4, 2, 16, 0.35, "gelu_erf", kv_from=kv1)
    expected = plain_head(x, w)
    torch.testing.assert_close(got, expected, rtol=1e-4, atol=1e-4 * float(expected.abs().max()))


# ---- a toy mixer with state of its own, defined here ------------------------------------------
@register_part("mixer", "toy_decay")
class ToyDecayMixer(Mixer):
    """s_t = decay * s_{t-1} + W h_t per request; adds s_t to the residual. Its state is one
    fp32 vector per request, kept in the engine's per-request state slots."""

    def __init__(self, spec, ctx, position=None):
        super().__init__(ctx)
        self.width = int(spec.width)
        self.decay = float(spec.decay)
        self.weight = self.add_param("mix.weight", (self.width, self.width), "matrix")

    def state_need(self):
        return StateNeed((self.width,), torch.float32)

    def forward(self, hidden, residual, step, cache):
        n = step.num_rows
        mixed = hidden[:n].float() @ self.weight.float().t()
        at = 0
        for rows, slot in zip(step.host_rows, step.host_state_slot):
            state = cache.state[slot]
            for r in range(at, at + rows):
                state.mul_(self.decay).add_(mixed[r])
                residual[r] += state
            at += rows


def plain_toy_layer(x, w, prefix, decay, act="gelu_tanh"):
    h = plain.layer_norm(x, w[prefix + "mixer_norm.weight"], w[prefix + "mixer_norm.bias"], 1e-5)
    mixed = h @ w[prefix + "mixer.mix.weight"].t()
    state = torch.zeros(x.shape[1])
    rows = []
    for t in range(x.shape[0]):
        state = decay * state + mixed[t]
        rows.append(x[t] + state)
    x = torch.stack(rows)
    h = plain.layer_norm(x, w[prefix + "feed_forward_norm.weight"],
                         w[prefix + "feed_forward_norm.bias"], 1e-5)
    inner = plain.gelu(h @ w[prefix + "feed_forward.up.weight"].t()
                       + w[prefix + "feed_forward.up.bias"], "gelu_new")
    return x + inner @ w[prefix + "feed_forward.down.weight"].t() + w[prefix + "feed_forward.down.bias"]


def test_a_toy_mixer_with_state_is_registered_built_and_stepped():
    width = 48
    norm = PartSpec("layer_norm", width=width, eps=1e-5, bias=True)
    toy = LayerSpec("pre_norm", PartSpec("toy_decay", width=width, decay=0.8),
                    PartSpec("dense", width=width, inner=64, activation="gelu_tanh", bias=True),
                    norm, norm)
    layers = [toy, attention_layer(width, 3, 3, 16, 0.25, 64)]
    spec = model_spec(layers, [Run(0), Run(1)], width, position_kind="none")
    core, w = core_of(spec, running=2)
    assert core.cache_plan.run_state[0] == StateNeed((width,), torch.float32)
    assert core.cache_plan.run_group == (None, 0)

    def expected_for(tokens):
        x = w["embedding.weight"][tokens]
        x = plain_toy_layer(x, w, "layers.0.", 0.8)
        x, _ = plain_attention_layer(x, w, "layers.1.", 3, 3, 16, 0.25, "gelu_tanh")
        return plain_head(x, w)

    first = [(3 * i + 2) % 61 for i in range(30)]
    second = [(11 * i + 5) % 61 for i in range(22)]
    # two requests interleaved, each in portions: the state persists between steps per request
    got_a = [core.step([StepEntry("a", first[:10], list(range(10)))]).cpu()]
    mixed = core.step([StepEntry("b", second[:5], list(range(5))),
                       StepEntry("a", first[10:11], [0])]).cpu()
    got_b = [mixed[:5]]
    got_a.append(mixed[5:])
    got_a.append(core.step([StepEntry("a", first[11:], list(range(19)))]).cpu())
    got_b.append(core.step([StepEntry("b", second[5:], list(range(17)))]).cpu())
    torch.testing.assert_close(torch.cat(got_a), expected_for(first), rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(torch.cat(got_b), expected_for(second), rtol=1e-4, atol=1e-4)
    # a new request that reuses a's slot starts from a zeroed state
    core.release("a")
    third = [(7 * i) % 61 for i in range(9)]
    got_c = core.step([StepEntry("c", third, list(range(9)))]).cpu()
    assert core.manager.row("c") == 0
    torch.testing.assert_close(got_c, expected_for(third), rtol=1e-4, atol=1e-4)


# ---- a toy feed-forward with routing and a toy rotary position encoding, defined here ----------
@register_part("feed_forward", "toy_routed")
class ToyRoutedFeedForward(FeedForward):
    """Top-1 routing over ``experts`` square matrices: residual += gate * (W_e h), with e the
    arg-max of the router's fp32 logits and gate its softmax probability."""

    def __init__(self, spec, ctx):
        super().__init__(ctx)
        self.width = int(spec.width)
        self.experts = int(spec.experts)
        self.router = self.add_param("router.weight", (self.experts, self.width), "matrix")
        self.weight = self.add_param("experts.weight", (self.experts * self.width, self.width),
                                     "matrix")

    def forward(self, hidden, residual, step):
        n = step.num_rows
        h = hidden[:n].float()
        prob = torch.softmax(h @ self.router.float().t(), dim=-1)
        gate, expert = prob.max(dim=-1)
        w = self.weight.float().view(self.experts, self.width, self.width)[expert]
        residual[:n] += gate[:, None] * torch.einsum("noi,ni->no", w, h)


@register_part("position", "toy_rotary")
class ToyRotary(PositionEncoding):
    """Rotates consecutive pairs of every head of the queries and keys by position * base **
    (-pair / pairs), in place, before the keys are cached."""

    def __init__(self, spec, ctx):
        super().__init__(ctx)
        self.head_dim = int(spec.head_dim)
        self.base = float(spec.base)

    def _angles(self, positions):
        pairs = self.head_dim // 2
        freq = self.base ** (-torch.arange(pairs, device=positions.device,
                                           dtype=torch.float32) / pairs)
        return positions.float()[:, None] * freq[None, :]

    def on_query_key(self, q, k, step):
        n = step.num_rows
        angle = self._angles(step.positions[:n])
        cos, sin = angle.cos()[:, None, :], angle.sin()[:, None, :]
        for t in (q, k):
            x = t[:n].float().reshape(n, -1, self.head_dim // 2, 2)
            a, b = x[..., 0], x[..., 1]
            turned = torch.stack([a * cos - b * sin, a * sin + b * cos], dim=-1)
            t[:n] = turned.reshape(n, -1).to(t.dtype)


def plain_rotate(x, head_dim, base):
    """[steps, heads, head_dim] rotated as ToyRotary does, position = row index."""
    pairs = head_dim // 2
    freq = base ** (-torch.arange(pairs, dtype=torch.float32) / pairs)
    angle = torch.arange(x.shape[0], dtype=torch.float32)[:, None] * freq[None, :]
    cos, sin = angle.cos()[:, None, :], angle.sin()[:, None, :]
    y = x.reshape(x.shape[0], x.shape[1], pairs, 2)
    return torch.stack([y[..., 0] * cos - y[..., 1] * sin, y[..., 0] * sin + y[..., 1] * cos],
                       dim=-1).reshape(x.shape)


def plain_rotary_routed_layer(x, w, prefix, heads, head_dim, scale, base, experts):
    steps, width = x.shape
    h = plain.layer_norm(x, w[prefix + "mixer_norm.weight"], w[prefix + "mixer_norm.bias"], 1e-5)
    qkv = h @ w[prefix + "mixer.qkv.weight"].t() + w[prefix + "mixer.qkv.bias"]
    q, k, v = (t.reshape(steps, heads, head_dim) for t in qkv.split(heads * head_dim, dim=-1))
    q, k = plain_rotate(q, head_dim, base), plain_rotate(k, head_dim, base)
    attended = plain.causal_attention(q, k, v, scale, 0).reshape(steps, heads * head_dim)
    x = x + attended @ w[prefix + "mixer.out.weight"].t() + w[prefix + "mixer.out.bias"]
    h = plain.layer_norm(x, w[prefix + "feed_forward_norm.weight"],
                         w[prefix + "feed_forward_norm.bias"], 1e-5)
    prob = torch.softmax(h @ w[prefix + "feed_forward.router.weight"].t(), dim=-1)
    gate, expert = prob.max(dim=-1)
    mats = w[prefix + "feed_forward.experts.weight"].view(experts, width, width)
    return x + gate[:, None] * torch.einsum("noi,ni->no", mats[expert], h)


def test_a_toy_routed_feed_forward_and_a_toy_rotary_encoding():
    """Another feed-forward kind and another position encoding, registered from this file:
    a layer with rotary attention and top-1 routing, then an ordinary layer (which the same
    encoding also rotates), whole, in portions and token by token over the paged cache."""
    width, heads, head_dim, experts, base = 48, 3, 16, 4, 50.0
    norm = PartSpec("layer_norm", width=width, eps=1e-5, bias=True)
    routed = LayerSpec("pre_norm",
                       PartSpec("attention", width=width, num_heads=heads, num_kv_heads=heads,
                                head_dim=head_dim, scale=0.3, window=0, bias=True),
                       PartSpec("toy_routed", width=width, experts=experts), norm, norm)
    spec = model_spec([routed], [Run(0)], width,
                      position_kind=PartSpec("toy_rotary", head_dim=head_dim, base=base))
    core, w = core_of(spec, running=2)
    tokens = [(5 * i + 1) % 61 for i in range(41)]

    x = w["embedding.weight"][tokens]
    x = plain_rotary_routed_layer(x, w, "layers.0.", heads, head_dim, 0.3, base, experts)
    expected = plain_head(x, w)
    whole = feed(core, "whole", tokens, [41])
    torch.testing.assert_close(whole, expected, rtol=1e-4, atol=1e-4)
    core.release("whole")
    cut = feed(core, "cut", tokens, [7, 2, 19] + [1] * 13)  # portions, then token by token
    torch.testing.assert_close(cut, expected, rtol=1e-4, atol=1e-4)


def test_an_unknown_part_kind_says_what_is_registered():
    from ayaka_b200.errors import ConfigError

    with pytest.raises(ConfigError) as caught:
        build_part("mixer", "mamba", PartSpec("mamba"), BuildContext(torch.float32, DEV))
    assert "attention" in str(caught.value) and "toy_decay" in str(caught.value)


def test_an_embedding_scale_and_a_logit_cap_are_parameters_of_the_parts():
    """What architectures other than GPT-2 do at the two ends of the model: the token rows
    times a factor (here sqrt(width)) before the positions are added, and the head's logits
    times a factor and squashed into (-cap, cap). Both are parameters of the embedding and
    head parts; a spec that sets them runs with no change to the package."""
    width, vocab = 48, 61
    scale, logit_scale, cap = math.sqrt(width), 0.5, 3.0
    spec = model_spec([attention_layer(width, 3, 3, 16, 0.25, 64)], [Run(0)], width, vocab=vocab)
    spec = dataclasses.replace(
        spec, embedding=PartSpec("token", vocab_size=vocab, width=width, scale=scale),
        head=PartSpec("linear", vocab_size=vocab, width=width, tied=True,
                      logit_scale=logit_scale, logit_softcap=cap))
    for dtype, tol in (("float32", 1e-4), ("bfloat16", 3e-2)):
        core, w = core_of(spec, dtype=dtype)
        tokens = [(5 * i + 1) % vocab for i in range(40)]
        x = w["embedding.weight"][tokens] * scale + w["position.weight"][:len(tokens)]
        x, _ = plain_attention_layer(x, w, "layers.0.", 3, 3, 16, 0.25, "gelu_tanh")
        expected = cap * torch.tanh(plain_head(x, w) * logit_scale / cap)
        got = feed(core, "s", tokens, [17, 1, 22])
        # (as in the engine tests: a fraction of the logit scale, which the cap bounds)
        torch.testing.assert_close(got, expected.float(), rtol=tol, atol=tol * cap)
        assert float(got.abs().max()) < cap
