"""Make the golden outputs: the reference's own GPT-2 code on tiny random models, on the CPU.

    python tests/golden/make_golden.py --reference PATH_TO_A_CHECKOUT_OF_gityuko-hb/ayaka

For each case below it draws random weights with this repository's random-weights mode
(checkpoint names and layout), loads them into the reference's ``GPT2LMHeadModel`` through
its own weight mapping, runs the token sequences through the reference's paged test driver
``run_paged`` (prompt in chunks, then token by token) and its ``compute_logits``, and stores
the token ids and float32 logits in ``tests/golden/<case>.npz``. ``tests/test_plain.py``
compares the plain implementation with these files. Case B runs with
``scale_attn_by_inverse_layer_idx`` false here because the reference ignores that key.
"""

from __future__ import annotations

import argparse
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))
sys.path.insert(0, str(HERE.parent))

from cases import CASES, case_config, case_sequences, case_state  # noqa: E402


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--reference", required=True)
    args = parser.parse_args()
    sys.dont_write_bytecode = True
    sys.path.insert(0, str(Path(args.reference) / "python"))
    sys.path.insert(0, str(Path(args.reference) / "tests" / "_support"))
    from ayaka.configs.model import ModelConfig
    from ayaka.models.gpt2 import GPT2LMHeadModel
    from ayaka.ops.backend import load_backend
    from ayaka.utils.dtypes import DType
    from gpt2_support import load_hf_state, run_paged

    for name in ("golden_a", "golden_b"):
        case = CASES[name]
        config_json = case_config(case)
        state = case_state(case)
        config = ModelConfig.from_hf_config(config_json)
        ops = load_backend(["torch"], device="cpu", dtype=DType.FP32)
        model = GPT2LMHeadModel(config, ops=ops, dtype=DType.FP32, device="cpu").eval()
        load_hf_state(model, state)
        sequences = [torch.tensor(ids) for ids in case_sequences(case)]
        prompts = [max(1, len(ids) - 3) for ids in sequences]
        with torch.inference_mode():
            hidden = run_paged(model, sequences, prompt_lengths=prompts, chunk=case["chunk"])
            logits = [model.compute_logits(h).float().numpy() for h in hidden]
        arrays = {}
        for index, (ids, values) in enumerate(zip(sequences, logits)):
            keep = sorted(set(range(0, len(ids), case["keep_every"])) | {len(ids) - 1})
            arrays[f"tokens_{index}"] = ids.numpy().astype(np.int32)
            arrays[f"rows_{index}"] = np.asarray(keep, dtype=np.int32)
            arrays[f"logits_{index}"] = values[keep].astype(np.float32)
        np.savez(HERE / f"{name}.npz", **arrays)
        print(name, {key: value.shape for key, value in arrays.items()})


if __name__ == "__main__":
    main()
