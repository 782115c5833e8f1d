"""Run the upstream project's own Qwen3 model on the CPU and store small outputs.

Usage (once; the outputs are committed beside this script):

    python tests/golden/make_golden.py --upstream-src <checkout>/src

It imports ``forge_engine.qwen3`` from the given source tree of
marcoharuni/forge-engine (the package is not installed, so the version lookup in its
``__init__`` is answered by a shim), builds ``Qwen3ForCausalLM`` for the tiny
configurations A, B and C (C has biases on q/k/v/o) of ``tests/plain_qwen3.py``, loads the seeded weights of
``plain_qwen3.seeded_weights`` into it by name and stores, per configuration,

* ``ids``            the token ids that were fed,
* ``logits``         upstream logits ``[T, vocab]`` (for the untied configuration B:
                     ``last_hidden_state @ lm_head.weight.T``, since upstream always ties),
* ``layer_<i>``      the hidden state after layer ``i``,
* ``chunked_logits`` the same tokens fed in portions 8, 8, 6, 2 through upstream's
                     tuple cache (``forward(chunk, past_key_values=...)``).

``tests/test_plain.py`` compares the plain implementation with these tensors.
"""

from __future__ import annotations

import argparse
import importlib.metadata
import sys
from pathlib import Path

import torch
from safetensors.torch import save_file

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))

import plain_qwen3 as plain  # noqa: E402


def import_upstream(src: str):
    real_version = importlib.metadata.version

    def version(name: str) -> str:
        if name == "forge-engine":
            return "0.0.0+source"
        return real_version(name)

    importlib.metadata.version = version
    sys.path.insert(0, src)
    from forge_engine import qwen3  # type: ignore

    return qwen3


def run(qwen3, raw: dict, seed: int, ids_seed: int, length: int) -> dict[str, torch.Tensor]:
    cfg = plain.PlainConfig.from_dict(raw)
    weights = plain.seeded_weights(cfg, seed)
    eos = raw["eos_token_id"]
    upstream_cfg = qwen3.Qwen3Config(
        vocab_size=cfg.vocab_size,
        hidden_size=cfg.hidden_size,
        intermediate_size=cfg.intermediate_size,
        num_hidden_layers=cfg.num_hidden_layers,
        num_attention_heads=cfg.num_attention_heads,
        num_key_value_heads=cfg.num_key_value_heads,
        head_dim=cfg.head_dim,
        max_position_embeddings=raw["max_position_embeddings"],
        rms_norm_eps=cfg.rms_norm_eps,
        rope_theta=cfg.rope_theta,
        eos_token_id=eos if isinstance(eos, int) else eos[0],
        tie_word_embeddings=True,
        attention_bias=cfg.attention_bias,
    )
    model = qwen3.Qwen3ForCausalLM(upstream_cfg).eval()
    state = {k: v for k, v in weights.items() if k != "lm_head.weight"}
    model.load_state_dict(state, strict=True)
    generator = torch.Generator().manual_seed(ids_seed)
    ids = torch.randint(0, cfg.vocab_size, (length,), generator=generator)

    def logits_of(output) -> torch.Tensor:
        if cfg.tie_word_embeddings:
            return output.logits[0]
        return (output.last_hidden_state[0] @ weights["lm_head.weight"].t()).float()

    out: dict[str, torch.Tensor] = {"ids": ids.to(torch.int32)}
    with torch.inference_mode():
        whole = model(input_ids=ids.unsqueeze(0))
        out["logits"] = logits_of(whole).contiguous()
        for index, hidden in enumerate(whole.layer_hidden_states):
            out[f"layer_{index}"] = hidden[0].contiguous()
        past = None
        rows = []
        start = 0
        for portion in (8, 8, 6, 2):
            chunk = ids[start : start + portion].unsqueeze(0)
            step = model(input_ids=chunk, past_key_values=past)
            past = step.past_key_values
            rows.append(logits_of(step))
            start += portion
        assert start == length
        out["chunked_logits"] = torch.cat(rows, dim=0).contiguous()
    return out


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--upstream-src", required=True)
    args = parser.parse_args()
    qwen3 = import_upstream(args.upstream_src)
    torch.manual_seed(0)
    for name, raw, seed, ids_seed in (
        ("tiny_a", plain.TINY_A, 0, 1),
        ("tiny_b", plain.TINY_B, 2, 3),
        ("tiny_c", plain.TINY_C, 5, 7),
    ):
        tensors = run(qwen3, raw, seed, ids_seed, 24)
        save_file(tensors, str(HERE / f"{name}.safetensors"))
        print(name, {k: tuple(v.shape) for k, v in tensors.items()})


if __name__ == "__main__":
    main()
