"""The plain GPT-2 of ``plain_gpt2.py`` with the roundings a bfloat16 engine makes.

The float64 oracle cannot see a bfloat16 fault smaller than bfloat16's own rounding noise,
which after a few layers is a few per cent of the logit scale. This variant computes every
product and sum in float64 like the oracle, but rounds to bfloat16 exactly where an engine
that keeps its activations in bfloat16 between kernels must: the normalised hidden state,
the fused query/key/value projection, the attention output, the activated feed-forward inner
state, the final normalised rows. The residual stream is never rounded (the engine keeps it
in float32 and adds into it inside the last product of each half), the softmax stays exact,
and the logits are not rounded (float32 out of the head). What is left between this and
the engine is the order of float32 sums and roundings that fall on the other side of a tie,
which is an order of magnitude below the rounding noise itself.

It shares no code with ``ayaka_b200``; formulas as in ``plain_gpt2.py`` (which cites the
reference's files and lines).
"""

from __future__ import annotations

import torch

import plain_gpt2 as plain


def bf16(x: torch.Tensor) -> torch.Tensor:
    """Round to the nearest bfloat16 (ties to even) and widen again."""
    return x.to(torch.bfloat16).to(x.dtype)


def attention_block(x: torch.Tensor, state: dict, block: str, heads: int, head_dim: int,
                    scale: float, round_weights: bool, reference_shift: float = 0.0
                    ) -> torch.Tensor:
    steps, hidden = x.shape
    qkv = bf16(plain.conv1d(x, state[f"{block}.attn.c_attn.weight"],
                            state[f"{block}.attn.c_attn.bias"]))
    q, k, v = (part.reshape(steps, heads, head_dim) for part in qkv.split(hidden, dim=-1))
    if round_weights:
        # a tensor-core kernel multiplies bfloat16 weights exp(s - reference) by the values
        # and divides by their exact sum afterwards; its reference is a running maximum,
        # here the row's maximum moved by ``reference_shift``
        scores = torch.einsum("thd,shd->hts", q, k) * scale
        hidden_keys = torch.arange(steps)[None, :] > torch.arange(steps)[:, None]
        scores = scores.masked_fill(hidden_keys[None], float("-inf"))
        raised = torch.exp(scores - scores.max(dim=-1, keepdim=True).values + reference_shift)
        attended = torch.einsum("hts,shd->thd", bf16(raised), v) / \
            raised.sum(dim=-1).t()[:, :, None]
    else:
        attended = plain.causal_attention(q, k, v, scale)
    attended = bf16(attended.reshape(steps, hidden))
    return plain.conv1d(attended, state[f"{block}.attn.c_proj.weight"],
                        state[f"{block}.attn.c_proj.bias"])


def mlp_block(x: torch.Tensor, state: dict, block: str, act: str) -> torch.Tensor:
    inner = bf16(plain.gelu(plain.conv1d(x, state[f"{block}.mlp.c_fc.weight"],
                                         state[f"{block}.mlp.c_fc.bias"]), act))
    return plain.conv1d(inner, state[f"{block}.mlp.c_proj.weight"],
                        state[f"{block}.mlp.c_proj.bias"])


def logits(state: dict, config: dict, tokens: torch.Tensor, round_weights: bool = False,
           reference_shift: float = 0.0) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence with bfloat16 activations between the parts.
    ``state`` holds bfloat16-representable values widened to float64."""
    s, p = plain.sizes(config), plain.prefix_of(state)
    steps = tokens.shape[0]
    x = plain.embed(state[f"{p}wte.weight"], state[f"{p}wpe.weight"], tokens,
                    torch.arange(steps))
    for layer in range(s["layers"]):
        block = f"{p}h.{layer}"
        normed = bf16(plain.layer_norm(x, state[f"{block}.ln_1.weight"],
                                       state[f"{block}.ln_1.bias"], s["eps"]))
        x = x + attention_block(normed, state, block, s["heads"], s["head_dim"],
                                plain.attention_scale(s["head_dim"], layer,
                                                      s["scale_by_layer"]), round_weights,
                                reference_shift)
        normed = bf16(plain.layer_norm(x, state[f"{block}.ln_2.weight"],
                                       state[f"{block}.ln_2.bias"], s["eps"]))
        x = x + mlp_block(normed, state, block, s["act"])
    final = bf16(plain.layer_norm(x, state[f"{p}ln_f.weight"], state[f"{p}ln_f.bias"],
                                  s["eps"]))
    head = state[f"{p}wte.weight"] if s["tied"] else state["lm_head.weight"]
    return final @ head.t()
