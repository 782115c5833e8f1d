"""Plain, slow Qwen3 dense decoder: whole sequences, no cache, one function per part.

This file is the yardstick the engine is measured against.  It shares no code with
the package: it only needs ``torch`` and a ``dict`` of tensors keyed by the
checkpoint's tensor names.  Every function restates one formula of the upstream
model file and cites it as ``path:line`` inside the upstream project
(marcoharuni/forge-engine).  ``tests/golden/make_golden.py`` ran the upstream
``Qwen3ForCausalLM`` on the CPU once and stored its outputs; ``test_plain.py``
compares this file with those stored outputs.

Two precisions:

* ``dtype=torch.float32`` - everything in 32-bit.
* ``dtype=torch.bfloat16`` - the upstream bfloat16 data flow: activations and
  weights in bfloat16, with the variance of the norms, the rotation angles and the
  softmax in 32-bit exactly where the upstream code has them.

Everything runs where the weights live: on the CPU for the tiny configurations, and - for
the checks at the benchmark's layer sizes, which would take minutes on the CPU - on the
GPU with plain torch operators (32-bit matrix products without any reduced-precision
mode; the caller switches TF32 off).  ``weights`` may be any mapping from tensor name to
tensor, also one that makes a tensor when it is asked for; only one layer's tensors are
held at a time.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
from torch import Tensor


@dataclass(frozen=True)
class PlainConfig:
    """The sizes and constants the formulas need (src/forge_engine/qwen3.py:18-34)."""

    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool
    attention_bias: bool = False
    sliding_window: int | None = None
    max_window_layers: int = 0

    @classmethod
    def from_dict(cls, raw: dict) -> "PlainConfig":
        return cls(
            vocab_size=int(raw["vocab_size"]),
            hidden_size=int(raw["hidden_size"]),
            intermediate_size=int(raw["intermediate_size"]),
            num_hidden_layers=int(raw["num_hidden_layers"]),
            num_attention_heads=int(raw["num_attention_heads"]),
            num_key_value_heads=int(raw["num_key_value_heads"]),
            head_dim=int(
                raw.get("head_dim", raw["hidden_size"] // raw["num_attention_heads"])
            ),
            rms_norm_eps=float(raw["rms_norm_eps"]),
            rope_theta=float(raw["rope_theta"]),
            tie_word_embeddings=bool(raw.get("tie_word_embeddings", False)),
            attention_bias=bool(raw.get("attention_bias", False)),
            sliding_window=(
                int(raw["sliding_window"])
                if raw.get("sliding_window") is not None
                and raw.get("use_sliding_window", True)
                else None
            ),
            max_window_layers=int(raw.get("max_window_layers", 0)),
        )

    def window_of_layer(self, index: int) -> int | None:
        """Upstream refuses any window (src/forge_engine/qwen3.py:44-45); with
        ``use_sliding_window`` the layers from ``max_window_layers`` on see only the
        last ``sliding_window`` keys (their own included).  This rests on the formula."""
        if self.sliding_window is None or index < self.max_window_layers:
            return None
        return self.sliding_window


def rms_norm(x: Tensor, weight: Tensor, eps: float) -> Tensor:
    """src/forge_engine/qwen3.py:99-105 - 32-bit variance, cast back, then weight."""
    dtype = x.dtype
    x32 = x.float()
    variance = x32.square().mean(dim=-1, keepdim=True)
    x32 = x32 * torch.rsqrt(variance + eps)
    return weight * x32.to(dtype)


def linear(x: Tensor, weight: Tensor, bias: Tensor | None = None) -> Tensor:
    """``nn.Linear`` with an ``[out, in]`` weight (src/forge_engine/qwen3.py:113-122)."""
    y = x @ weight.t()
    return y if bias is None else y + bias


def rotary_tables(
    positions: Tensor, head_dim: int, theta: float, dtype: torch.dtype
) -> tuple[Tensor, Tensor]:
    """src/forge_engine/qwen3.py:345-363 - angles in 32-bit, rounded to ``dtype``."""
    frequencies = 1.0 / (
        theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim)
    ).to(positions.device)
    phases = positions.float().unsqueeze(-1) * frequencies
    embeddings = torch.cat((phases, phases), dim=-1)
    return embeddings.cos().to(dtype), embeddings.sin().to(dtype)


def rotate_half(x: Tensor) -> Tensor:
    """src/forge_engine/qwen3.py:366-369 - pairs element j with j + D/2."""
    first, second = x.chunk(2, dim=-1)
    return torch.cat((-second, first), dim=-1)


def apply_rotary(x: Tensor, cosine: Tensor, sine: Tensor) -> Tensor:
    """src/forge_engine/qwen3.py:372-381 - ``x`` is [heads, T, D]; tables are [T, D]."""
    return x * cosine.unsqueeze(0) + rotate_half(x) * sine.unsqueeze(0)


def causal_mask(length: int, dtype: torch.dtype, window: int | None = None, device=None) -> Tensor:
    """src/forge_engine/qwen3.py:384-406 with no past: key j is seen by query i iff j <= i
    (and, with a window, i - j < window)."""
    positions = torch.arange(length, device=device)
    allowed = positions.unsqueeze(0) <= positions.unsqueeze(1)
    if window is not None:
        allowed = allowed & (positions.unsqueeze(1) - positions.unsqueeze(0) < window)
    mask = torch.zeros((length, length), dtype=dtype, device=device)
    return mask.masked_fill(~allowed, torch.finfo(dtype).min)


def attention(
    x: Tensor,
    weights: dict[str, Tensor],
    prefix: str,
    cfg: PlainConfig,
    window: int | None = None,
) -> Tensor:
    """Causal grouped-query attention of one layer over a whole sequence.

    src/forge_engine/qwen3.py:141-207: projections, per-head q/k RMSNorm over
    head_dim (one weight shared by all heads), rotation of q and k, scores in the
    model dtype scaled by head_dim**-0.5, additive causal mask, softmax in 32-bit
    cast back to the model dtype, value product, output projection.
    """
    length = x.shape[0]
    nq, nkv, d = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    groups = nq // nkv

    def bias(name: str) -> Tensor | None:
        return weights[f"{prefix}.{name}.bias"] if cfg.attention_bias else None

    q = linear(x, weights[f"{prefix}.q_proj.weight"], bias("q_proj")).view(length, nq, d)
    k = linear(x, weights[f"{prefix}.k_proj.weight"], bias("k_proj")).view(length, nkv, d)
    v = linear(x, weights[f"{prefix}.v_proj.weight"], bias("v_proj")).view(length, nkv, d)
    q = rms_norm(q, weights[f"{prefix}.q_norm.weight"], cfg.rms_norm_eps).transpose(0, 1)
    k = rms_norm(k, weights[f"{prefix}.k_norm.weight"], cfg.rms_norm_eps).transpose(0, 1)
    v = v.transpose(0, 1)
    cosine, sine = rotary_tables(torch.arange(length, device=x.device), d, cfg.rope_theta, x.dtype)
    q = apply_rotary(q, cosine, sine)
    k = apply_rotary(k, cosine, sine)
    k = k.repeat_interleave(groups, dim=0)
    v = v.repeat_interleave(groups, dim=0)
    scores = torch.matmul(q, k.transpose(1, 2)) * d**-0.5
    scores = scores + causal_mask(length, scores.dtype, window, x.device)
    probabilities = torch.softmax(scores, dim=-1, dtype=torch.float32).to(q.dtype)
    out = torch.matmul(probabilities, v).transpose(0, 1).reshape(length, nq * d)
    return linear(out, weights[f"{prefix}.o_proj.weight"], bias("o_proj"))


def feed_forward(x: Tensor, weights: dict[str, Tensor], prefix: str) -> Tensor:
    """src/forge_engine/qwen3.py:225-227 - down(silu(gate(x)) * up(x)), no biases."""
    gate = linear(x, weights[f"{prefix}.gate_proj.weight"])
    up = linear(x, weights[f"{prefix}.up_proj.weight"])
    return linear(torch.nn.functional.silu(gate) * up, weights[f"{prefix}.down_proj.weight"])


def decoder_layer(
    h: Tensor, weights: dict[str, Tensor], index: int, cfg: PlainConfig
) -> Tensor:
    """src/forge_engine/qwen3.py:241-261 - pre-norm block with two residual sums."""
    prefix = f"model.layers.{index}"
    normed = rms_norm(h, weights[f"{prefix}.input_layernorm.weight"], cfg.rms_norm_eps)
    h = h + attention(
        normed, weights, f"{prefix}.self_attn", cfg, cfg.window_of_layer(index)
    )
    # src/forge_engine/kernels/__init__.py:12-26: sum, then the same RMSNorm.
    normed = rms_norm(
        h, weights[f"{prefix}.post_attention_layernorm.weight"], cfg.rms_norm_eps
    )
    return h + feed_forward(normed, weights, f"{prefix}.mlp")


class _Cast:
    """``weights`` with every tensor converted to ``dtype`` when it is looked up."""

    def __init__(self, weights, dtype: torch.dtype) -> None:
        self.weights, self.dtype = weights, dtype

    def __getitem__(self, name: str) -> Tensor:
        return self.weights[name].to(self.dtype)


def hidden_states(
    ids: Tensor, weights: dict[str, Tensor], cfg: PlainConfig, dtype: torch.dtype
) -> tuple[Tensor, list[Tensor]]:
    """Embedding, all layers, final norm (src/forge_engine/qwen3.py:325-335)."""
    w = _Cast(weights, dtype)
    table = w["model.embed_tokens.weight"]
    h = table[ids.long().to(table.device)]
    del table
    per_layer = []
    for index in range(cfg.num_hidden_layers):
        h = decoder_layer(h, w, index, cfg)
        per_layer.append(h)
    return rms_norm(h, w["model.norm.weight"], cfg.rms_norm_eps), per_layer


def forward_logits(
    ids: Tensor | list[int],
    weights: dict[str, Tensor],
    cfg: PlainConfig,
    dtype: torch.dtype = torch.float32,
) -> Tensor:
    """Logits ``[T, vocab]`` in 32-bit for one whole sequence.

    src/forge_engine/qwen3.py:336 multiplies by the embedding table (tied).  With
    ``tie_word_embeddings`` false the table ``lm_head.weight`` stands in its place;
    the upstream project has no such tensor, so that case rests on the formula.
    """
    ids = torch.as_tensor(ids, dtype=torch.long)
    last, _ = hidden_states(ids, weights, cfg, dtype)
    name = "model.embed_tokens.weight" if cfg.tie_word_embeddings else "lm_head.weight"
    return linear(last, weights[name].to(dtype)).float()


# ---------------------------------------------------------------------------
# sampling
# ---------------------------------------------------------------------------


def filter_logits(
    logits: Tensor,
    temperature: float,
    top_k: int | None = None,
    top_p: float = 1.0,
    min_p: float = 0.0,
) -> Tensor:
    """src/forge_engine/sampling.py:83-140 - temperature, top-k, top-p, min-p in that order.

    Returns the filtered, shifted logits; ``softmax`` of them is the distribution a
    token is drawn from.
    """
    x = logits.float()
    x = (x - x.max(dim=-1, keepdim=True).values) / temperature
    neg = float("-inf")
    if top_k is not None and top_k < x.shape[-1]:
        values, indices = torch.topk(x, k=top_k, dim=-1)
        x = torch.full_like(x, neg).scatter(-1, indices, values)
    if top_p < 1.0:
        sorted_x, order = torch.sort(x, dim=-1, descending=True)
        probabilities = torch.softmax(sorted_x, dim=-1, dtype=torch.float32)
        remove = probabilities.cumsum(dim=-1) > top_p
        remove[..., 1:] = remove[..., :-1].clone()
        remove[..., 0] = False
        sorted_x = sorted_x.masked_fill(remove, neg)
        x = torch.full_like(x, neg).scatter(-1, order, sorted_x)
    if min_p > 0.0:
        probabilities = torch.softmax(x, dim=-1, dtype=torch.float32)
        threshold = probabilities.max(dim=-1, keepdim=True).values
        x = x.masked_fill(probabilities < threshold * min_p, neg)
    return x


def greedy(logits: Tensor) -> Tensor:
    """src/forge_engine/sampling.py:71-72."""
    return logits.argmax(dim=-1)


def greedy_generate(
    prompt: list[int],
    steps: int,
    weights: dict[str, Tensor],
    cfg: PlainConfig,
    dtype: torch.dtype = torch.float32,
) -> list[int]:
    """Recompute the whole sequence for every new token (no cache) and take argmax."""
    ids = list(prompt)
    out = []
    for _ in range(steps):
        token = int(greedy(forward_logits(ids, weights, cfg, dtype)[-1:]).item())
        out.append(token)
        ids.append(token)
    return out


# ---------------------------------------------------------------------------
# seeded weights and the two tiny configurations used throughout the tests
# ---------------------------------------------------------------------------

TINY_A = {
    "architectures": ["Qwen3ForCausalLM"],
    "model_type": "qwen3",
    "hidden_act": "silu",
    "vocab_size": 256,
    "hidden_size": 64,
    "intermediate_size": 128,
    "num_hidden_layers": 2,
    "num_attention_heads": 4,
    "num_key_value_heads": 2,
    "head_dim": 16,
    "max_position_embeddings": 4096,
    "rms_norm_eps": 1e-6,
    "rope_theta": 10000.0,
    "tie_word_embeddings": True,
    "attention_bias": False,
    "sliding_window": None,
    "eos_token_id": 255,
}

TINY_B = {
    "architectures": ["Qwen3ForCausalLM"],
    "model_type": "qwen3",
    "hidden_act": "silu",
    "vocab_size": 384,
    "hidden_size": 96,
    "intermediate_size": 200,
    "num_hidden_layers": 3,
    "num_attention_heads": 8,
    "num_key_value_heads": 2,
    "head_dim": 32,
    "max_position_embeddings": 8192,
    "rms_norm_eps": 1e-5,
    "rope_theta": 1000000.0,
    "tie_word_embeddings": False,
    "attention_bias": False,
    "sliding_window": None,
    "eos_token_id": [382, 383],
}

# Same as B but with biases on q/k/v/o, an odd number of heads per group and a
# vocabulary that is not a multiple of 8.
TINY_C = dict(
    TINY_B,
    vocab_size=331,
    hidden_size=80,
    num_attention_heads=6,
    num_key_value_heads=3,
    head_dim=48,
    intermediate_size=136,
    num_hidden_layers=2,
    attention_bias=True,
    rope_theta=50000.0,
    rms_norm_eps=3e-6,
    eos_token_id=[329, 330],
)


# Three layers, the last two windowed; nothing is a power of two.
TINY_D = dict(
    TINY_A,
    vocab_size=203,
    hidden_size=72,
    intermediate_size=88,
    num_hidden_layers=3,
    num_attention_heads=6,
    num_key_value_heads=2,
    head_dim=16,
    rms_norm_eps=2e-6,
    rope_theta=20000.0,
    tie_word_embeddings=False,
    use_sliding_window=True,
    sliding_window=11,
    max_window_layers=1,
    eos_token_id=202,
)


# Head size 64 (the tensor-memory prefill kernel and the TMA decode kernel take it), two
# heads per kv head, the second layer windowed with a window that ends inside a key tile.
TINY_E = dict(
    TINY_A,
    vocab_size=311,
    hidden_size=96,
    intermediate_size=144,
    num_hidden_layers=2,
    num_attention_heads=4,
    num_key_value_heads=2,
    head_dim=64,
    rms_norm_eps=1e-5,
    rope_theta=100000.0,
    use_sliding_window=True,
    sliding_window=70,
    max_window_layers=1,
    eos_token_id=310,
)


def tensor_shapes(cfg: PlainConfig) -> dict[str, tuple[int, ...]]:
    """Tensor names and shapes of a checkpoint (src/forge_engine/weights.py:253-282)."""
    h, i = cfg.hidden_size, cfg.intermediate_size
    q = cfg.num_attention_heads * cfg.head_dim
    kv = cfg.num_key_value_heads * cfg.head_dim
    shapes: dict[str, tuple[int, ...]] = {
        "model.embed_tokens.weight": (cfg.vocab_size, h),
        "model.norm.weight": (h,),
    }
    for layer in range(cfg.num_hidden_layers):
        p = f"model.layers.{layer}"
        shapes[f"{p}.input_layernorm.weight"] = (h,)
        shapes[f"{p}.post_attention_layernorm.weight"] = (h,)
        shapes[f"{p}.self_attn.q_norm.weight"] = (cfg.head_dim,)
        shapes[f"{p}.self_attn.k_norm.weight"] = (cfg.head_dim,)
        shapes[f"{p}.self_attn.q_proj.weight"] = (q, h)
        shapes[f"{p}.self_attn.k_proj.weight"] = (kv, h)
        shapes[f"{p}.self_attn.v_proj.weight"] = (kv, h)
        shapes[f"{p}.self_attn.o_proj.weight"] = (h, q)
        if cfg.attention_bias:
            shapes[f"{p}.self_attn.q_proj.bias"] = (q,)
            shapes[f"{p}.self_attn.k_proj.bias"] = (kv,)
            shapes[f"{p}.self_attn.v_proj.bias"] = (kv,)
            shapes[f"{p}.self_attn.o_proj.bias"] = (h,)
        shapes[f"{p}.mlp.gate_proj.weight"] = (i, h)
        shapes[f"{p}.mlp.up_proj.weight"] = (i, h)
        shapes[f"{p}.mlp.down_proj.weight"] = (h, i)
    if not cfg.tie_word_embeddings:
        shapes["lm_head.weight"] = (cfg.vocab_size, h)
    return shapes


def seeded_weights(
    cfg: PlainConfig, seed: int, std: float = 0.02, round_to_bf16: bool = True
) -> dict[str, Tensor]:
    """Matrices N(0, std), norm weights 1 + N(0, 0.1), biases N(0, std); fixed name order.

    ``round_to_bf16`` rounds every value to a bfloat16-representable number (still
    stored as float32), so that the 32-bit and the bfloat16 run see the same model.
    """
    generator = torch.Generator().manual_seed(seed)
    weights = {}
    for name, shape in tensor_shapes(cfg).items():
        noise = torch.randn(shape, generator=generator, dtype=torch.float32)
        value = 1.0 + 0.1 * noise if "norm" in name else std * noise
        weights[name] = value.bfloat16().float() if round_to_bf16 else value
    return weights
