"""Compare the plain implementation (tests/plain_llama.py) once with the reference's own model
code on the CPU, and store the reference's outputs next to this script.

    PYTHONPATH=<reference checkout>:<this repository> python tests/golden/make_golden.py

For each tiny configuration the reference's ``LlamaForCausalLM`` (engine/model/llama.py) gets
the weights of ``tests.helpers.make_weights`` (upcast to 32-bit; the tied head is tied by
hand, since its constructor does not tie) and computes the logits of one random sequence
without a cache.  The script asserts that the plain implementation agrees to 1e-5 and writes
``golden_<name>.npz`` (token ids and the reference's logits, 32-bit).
``tests/test_plain_llama.py`` checks the plain implementation against these files, so the
anchor holds where the reference is not installed.
"""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from tests import helpers, plain_llama  # noqa: E402
from tests.tiny_configs import TINY_A, TINY_B, TINY_C  # noqa: E402


def main() -> None:
    from engine.config import ModelConfig  # the reference
    from engine.model.llama import LlamaForCausalLM

    for name, cfg, length in (("A", TINY_A, 40), ("B", TINY_B, 90), ("C", TINY_C, 50)):
        weights = helpers.make_weights(cfg, seed=ord(name))
        ids = helpers.random_tokens(cfg, length, 1000 + ord(name))
        model = LlamaForCausalLM(ModelConfig.from_dict(cfg)).float().eval()
        state = {k: v.float() for k, v in weights.items()}
        if cfg.get("tie_word_embeddings"):
            state["lm_head.weight"] = state["model.embed_tokens.weight"]
        model.load_state_dict(state, strict=True)
        with torch.no_grad():
            t = torch.tensor([ids])
            ref = model(t, torch.arange(length)[None])[0]
        mine = plain_llama.logits_for(cfg, weights, ids)
        diff = float((ref - mine).abs().max())
        assert diff < 1e-5, f"tiny {name}: plain implementation differs from the reference by {diff}"
        # Keep the files small: every position's logits at a stride of the vocabulary plus
        # the full rows of three positions.
        keep_rows = [0, length // 2, length - 1]
        np.savez_compressed(
            Path(__file__).with_name(f"golden_{name}.npz"),
            token_ids=np.asarray(ids, dtype=np.int32),
            rows=np.asarray(keep_rows, dtype=np.int32),
            row_logits=ref[keep_rows].numpy().astype(np.float32),
            strided_logits=ref[:, ::7].numpy().astype(np.float32),
        )
        print(f"tiny {name}: max |reference - plain| = {diff:.2e}; wrote golden_{name}.npz")


if __name__ == "__main__":
    main()
