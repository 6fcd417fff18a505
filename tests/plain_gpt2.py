"""A plain, slow GPT-2: whole sequences, no cache, one function per part, CPU torch.

Written from the reference's formulas (gityuko-hb/ayaka; every function cites the file and
lines it restates) and shares no code with ``ayaka_b200``: it reads a checkpoint-named state
dict in checkpoint layout (Conv1D weights are ``[in, out]``) and a plain dict of
``config.json`` keys. ``tests/golden`` holds outputs of the reference's own model code on
tiny random models; ``test_plain_matches_golden`` compares this file with them, so the
formulas here are anchored on the reference's code, except
``scale_attn_by_inverse_layer_idx``, which the reference does not implement and which rests
on the formula alone.

Precision: every function computes in the dtype of its inputs; tests pass float32 or
float64 tensors.
"""

from __future__ import annotations

import math

import torch

# ---------------------------------------------------------------------------------------------
# configuration keys (python/ayaka/configs/model.py:182-191, 350-354, 361-371)


def cfg(config: dict, *names: str):
    for name in names:
        if config.get(name) is not None:
            return config[name]
    raise KeyError(names[0])


def sizes(config: dict) -> dict:
    hidden = cfg(config, "n_embd", "hidden_size")
    heads = cfg(config, "n_head", "num_attention_heads")
    inner = config.get("n_inner") or config.get("intermediate_size") or 4 * hidden
    return {
        "hidden": hidden, "heads": heads, "head_dim": config.get("head_dim") or hidden // heads,
        "inner": inner, "layers": cfg(config, "n_layer", "num_hidden_layers"),
        "eps": cfg(config, "layer_norm_epsilon", "layer_norm_eps"),
        "act": cfg(config, "activation_function", "hidden_act"),
        "scale_by_layer": bool(config.get("scale_attn_by_inverse_layer_idx", False)),
        "tied": bool(config.get("tie_word_embeddings", True)),
        "vocab": config["vocab_size"], "positions": cfg(config, "n_positions",
                                                        "max_position_embeddings"),
    }


def prefix_of(state: dict) -> str:
    return "transformer." if "transformer.wte.weight" in state else ""


# ---------------------------------------------------------------------------------------------
# parts


def embed(wte: torch.Tensor, wpe: torch.Tensor, tokens: torch.Tensor,
          positions: torch.Tensor) -> torch.Tensor:
    """x[i] = wte[token[i]] + wpe[position[i]] (python/ayaka/models/gpt2.py:175)."""
    return wte[tokens] + wpe[positions]


def layer_norm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor,
               eps: float) -> torch.Tensor:
    """(x - mean) / sqrt(biased var + eps) * weight + bias over the last dimension
    (python/ayaka/layers/norm.py:59-100, python/ayaka/ops/backends/torch/norm.py:18-38)."""
    mean = x.mean(dim=-1, keepdim=True)
    centred = x - mean
    var = (centred * centred).mean(dim=-1, keepdim=True)
    return centred / torch.sqrt(var + eps) * weight + bias


def conv1d(x: torch.Tensor, weight_in_out: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """y = x @ W + b with W stored [in, out] (python/ayaka/models/gpt2.py:14-18;
    python/ayaka/layers/linear.py:55-59 after the transposition of :124-129)."""
    return x @ weight_in_out + bias


def gelu(x: torch.Tensor, name: str) -> torch.Tensor:
    """tanh form for gelu_new / gelu_pytorch_tanh, erf form for gelu
    (python/ayaka/models/gpt2.py:47, python/ayaka/ops/backends/torch/activation.py:18-36)."""
    if name in ("gelu_new", "gelu_pytorch_tanh"):
        inner = math.sqrt(2.0 / math.pi) * (x + 0.044715 * x * x * x)
        return 0.5 * x * (1.0 + torch.tanh(inner))
    if name == "gelu":
        return 0.5 * x * (1.0 + torch.erf(x / math.sqrt(2.0)))
    raise ValueError(name)


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                     window: int = 0) -> torch.Tensor:
    """softmax(scale * q k^T, masked to keys 0..own position) v per head; q, k, v are
    [T, heads, head_dim] (python/ayaka/ops/attention.py:15-24, 133-137; mask and fp32 softmax
    python/ayaka/ops/backends/torch/attention.py:220-233). ``window`` > 0 keeps only the
    last ``window`` keys of each row (not a GPT-2 option; used to test the kernel)."""
    steps = q.shape[0]
    scores = torch.einsum("thd,shd->hts", q, k) * scale
    row = torch.arange(steps)[:, None]
    col = torch.arange(steps)[None, :]
    hidden = col > row
    if window > 0:
        hidden = hidden | (col < row - window + 1)
    scores = scores.masked_fill(hidden[None], float("-inf"))
    weights = torch.softmax(scores, dim=-1)
    return torch.einsum("hts,shd->thd", weights, v)


def attention_block(x: torch.Tensor, state: dict, block: str, heads: int, head_dim: int,
                    scale: float) -> torch.Tensor:
    """Fused projection with columns q | k | v, heads split by column ranges, attention,
    output projection (python/ayaka/layers/attention/dense.py:101-125)."""
    steps, hidden = x.shape
    qkv = conv1d(x, state[f"{block}.attn.c_attn.weight"], state[f"{block}.attn.c_attn.bias"])
    q, k, v = (part.reshape(steps, heads, head_dim) for part in qkv.split(hidden, dim=-1))
    attended = causal_attention(q, k, v, scale).reshape(steps, hidden)
    return conv1d(attended, state[f"{block}.attn.c_proj.weight"],
                  state[f"{block}.attn.c_proj.bias"])


def mlp_block(x: torch.Tensor, state: dict, block: str, act: str) -> torch.Tensor:
    """down(act(up(x))) (python/ayaka/layers/ffn/dense.py:55-57)."""
    inner = gelu(conv1d(x, state[f"{block}.mlp.c_fc.weight"], state[f"{block}.mlp.c_fc.bias"]),
                 act)
    return conv1d(inner, state[f"{block}.mlp.c_proj.weight"], state[f"{block}.mlp.c_proj.bias"])


def attention_scale(head_dim: int, layer: int, scale_by_layer: bool) -> float:
    """head_dim ** -0.5 (python/ayaka/layers/attention/dense.py:77); divided by layer + 1
    when scale_attn_by_inverse_layer_idx is set (formula only: the reference ignores it)."""
    scale = head_dim ** -0.5
    return scale / (layer + 1) if scale_by_layer else scale


def hidden_states(state: dict, config: dict, tokens: torch.Tensor) -> torch.Tensor:
    """Final hidden states [T, hidden] of one whole sequence
    (python/ayaka/models/gpt2.py:99-101, 170-178)."""
    s, p = sizes(config), prefix_of(state)
    steps = tokens.shape[0]
    x = embed(state[f"{p}wte.weight"], state[f"{p}wpe.weight"], tokens, torch.arange(steps))
    for layer in range(s["layers"]):
        block = f"{p}h.{layer}"
        normed = layer_norm(x, state[f"{block}.ln_1.weight"], state[f"{block}.ln_1.bias"],
                            s["eps"])
        x = x + attention_block(normed, state, block, s["heads"], s["head_dim"],
                                attention_scale(s["head_dim"], layer, s["scale_by_layer"]))
        normed = layer_norm(x, state[f"{block}.ln_2.weight"], state[f"{block}.ln_2.bias"],
                            s["eps"])
        x = x + mlp_block(normed, state, block, s["act"])
    return layer_norm(x, state[f"{p}ln_f.weight"], state[f"{p}ln_f.bias"], s["eps"])


def logits(state: dict, config: dict, tokens: torch.Tensor) -> torch.Tensor:
    """Logits [T, vocab] at every position: hidden @ wte^T, no bias, or @ lm_head^T when the
    head is not tied (python/ayaka/models/gpt2.py:165-182,
    python/ayaka/layers/embedding/token.py:81)."""
    s, p = sizes(config), prefix_of(state)
    head = state[f"{p}wte.weight"] if s["tied"] else state["lm_head.weight"]
    return hidden_states(state, config, tokens) @ head.t()


def cast_state(state: dict, dtype: torch.dtype) -> dict:
    return {name: tensor.to(dtype) for name, tensor in state.items()}


# ---------------------------------------------------------------------------------------------
# sampling (python/ayaka/ops/sampling.py:22-61, python/ayaka/sampling/rng.py:29-117)

_WORD = 0xFFFFFFFF


def philox4x32_10(counter: tuple[int, int, int, int], key: tuple[int, int]) -> tuple[int, ...]:
    """Philox-4x32 with 10 rounds on Python integers (python/ayaka/sampling/rng.py:40-73)."""
    c0, c1, c2, c3 = counter
    k0, k1 = key
    for round_index in range(10):
        if round_index:
            k0 = (k0 + 0x9E3779B9) & _WORD
            k1 = (k1 + 0xBB67AE85) & _WORD
        p0 = 0xD2511F53 * c0
        p1 = 0xCD9E8D57 * c2
        c0, c1, c2, c3 = (p1 >> 32) ^ c1 ^ k0, p1 & _WORD, (p0 >> 32) ^ c3 ^ k1, p0 & _WORD
    return c0, c1, c2, c3


def draw_uniform(seed: int, position: int, stream: int = 0, sequence: int = 0) -> float:
    """u in [0, 1) with 24 bits for the token produced at ``position``
    (python/ayaka/sampling/rng.py:76-99)."""
    words = philox4x32_10((position & _WORD, position >> 32, stream, sequence),
                          (seed & _WORD, seed >> 32))
    return (words[0] >> 8) / float(1 << 24)


def argmax_smallest_id(row: torch.Tensor) -> int:
    """Largest logit, smallest id on a tie (python/ayaka/ops/backends/torch/sampling.py:
    119-127)."""
    best = row.max()
    return int(torch.nonzero(row == best)[0, 0])


def sample_token(row: torch.Tensor, temperature: float, u: float, top_k: int = 0,
                 top_p: float = 1.0, min_p: float = 0.0) -> int:
    """Temperature, top-k, top-p, min-p and the inverse CDF over the canonical order
    (python/ayaka/ops/sampling.py:44-57; python/ayaka/ops/backends/torch/sampling.py:
    156-180). Computed in float64 so that it is an oracle, not a twin, of the kernel."""
    if temperature <= 0:
        return argmax_smallest_id(row)
    x = row.double() / temperature
    sorted_x, order = torch.sort(x, descending=True, stable=True)
    vocab = x.shape[0]
    rank = torch.arange(vocab)
    keep = torch.ones(vocab, dtype=torch.bool) if top_k <= 0 else rank < top_k
    p = torch.softmax(torch.where(keep, sorted_x, torch.tensor(-math.inf, dtype=x.dtype)), dim=0)
    cumulative = torch.cumsum(p, dim=0)
    before = torch.cat([torch.zeros(1, dtype=p.dtype), cumulative[:-1]])
    keep = keep & ((before < top_p) | (rank == 0))
    keep = keep & (p >= min_p * p[0])
    kept = torch.where(keep, p, torch.zeros_like(p))
    cdf = torch.cumsum(kept, dim=0)
    first = int((cdf <= u * cdf[-1]).sum())
    last = max(int((kept > 0).sum()) - 1, 0)
    return int(order[min(first, last)])


def adjust_logits(row: torch.Tensor, prompt: list[int], output: list[int], *,
                  repetition: float = 1.0, frequency: float = 0.0, presence: float = 0.0,
                  bias: dict[int, float] | None = None, allowed: set[int] | None = None,
                  banned: set[int] | None = None) -> torch.Tensor:
    """What a request may have done to its logits before the draw, in the reference's order
    (python/ayaka/ops/sampling.py:10-20): the mask of allowed and banned ids
    (python/ayaka/sampling/logits.py:176-214), the additive bias (python/ayaka/ops/backends/
    torch/sampling.py:203-213), then the penalties (python/ayaka/ops/sampling.py:176-200):
    x / r or x * r where the token occurs in prompt or output, minus f per occurrence in the
    output, minus s where it occurs in the output."""
    x = row.clone()
    vocab = x.shape[0]
    if allowed is not None:
        keep = torch.zeros(vocab, dtype=torch.bool)
        keep[sorted(allowed)] = True
        x[~keep] = -math.inf
    for token in banned or ():
        x[token] = -math.inf
    for token, value in (bias or {}).items():
        x[token] = x[token] + value
    seen = torch.zeros(vocab, dtype=torch.bool)
    seen[list(prompt) + list(output)] = True
    count = torch.zeros(vocab, dtype=x.dtype)
    for token in output:
        count[token] += 1
    x = torch.where(seen, torch.where(x > 0, x / repetition, x * repetition), x)
    x = x - frequency * count
    x = x - presence * (count > 0).to(x.dtype)
    return x


def greedy_generate(state: dict, config: dict, prompt: list[int], steps: int) -> list[int]:
    """Greedy continuation by rerunning the whole sequence each step, no cache
    (tests/_support/tiny_model.py:225-238 does the same in the reference)."""
    tokens = list(prompt)
    out = []
    for _ in range(steps):
        row = logits(state, config, torch.tensor(tokens))[-1]
        token = argmax_smallest_id(row)
        out.append(token)
        tokens.append(token)
    return out
