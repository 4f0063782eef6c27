"""Makes the golden logits under tests/golden/ from the REFERENCE's own model code.

Run once, on the CPU, where a checkout of ashwinsreedhar28/emberserve is importable:

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py /path/to/emberserve-checkout

For Tiny A and Tiny B it draws weights with this package's random-weights mode (stored in
float32), copies the tensors into the reference's ``Qwen2ForCausalLM`` through its
``load_hf_state_dict`` (emberserve/model/weights.py:202-209), runs its
``forward_logits_all`` with its naive attention backend (emberserve/attn/naive.py) on one
sequence, and stores the float32 logits together with the weights themselves
(``<name>_weights.safetensors``, float32, a few hundred KB), so that the comparison never
depends on what a later torch draws from the same seed.  The weights are copied into the
reference's model, never re-drawn: its own random initialisation draws in another order.
"""

from __future__ import annotations

import hashlib
import json
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))
sys.path.insert(0, str(HERE.parent))

from tiny_configs import ALL, SEEDS  # noqa: E402

from emberserve_b200.registry import build_decoder  # noqa: E402
from emberserve_b200.weights.loader import random_checkpoint  # noqa: E402
from emberserve_b200.weights.safetensors_io import write_safetensors  # noqa: E402

CASES = {"tiny_a": 17, "tiny_b": 40}  # sequence lengths


def checksum(tensors: dict[str, torch.Tensor]) -> str:
    h = hashlib.sha256()
    for name in sorted(tensors):
        h.update(name.encode())
        h.update(tensors[name].contiguous().view(torch.uint8).numpy().tobytes())
    return h.hexdigest()


def token_ids(name: str, n: int, vocab: int) -> list[int]:
    g = torch.Generator().manual_seed(1000 + SEEDS[name])
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def main() -> None:
    ref_root = sys.argv[1]
    sys.path.insert(0, ref_root)
    from emberserve.attn.base import AttnMetadata
    from emberserve.attn.naive import NaiveAttentionBackend
    from emberserve.config import ModelConfig as RefConfig
    from emberserve.model.qwen2 import Qwen2ForCausalLM
    from emberserve.model.weights import load_hf_state_dict

    meta_out = {}
    for name, n in CASES.items():
        cfg = ALL[name]
        tensors = random_checkpoint(build_decoder(cfg), SEEDS[name], store_dtype=torch.float32)
        ref_cfg = RefConfig(
            vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size,
            intermediate_size=cfg.intermediate_size, num_hidden_layers=cfg.num_hidden_layers,
            num_attention_heads=cfg.num_attention_heads, num_key_value_heads=cfg.num_key_value_heads,
            max_position_embeddings=cfg.max_position_embeddings, rms_norm_eps=cfg.rms_norm_eps,
            rope_theta=cfg.rope_theta, tie_word_embeddings=cfg.tie_word_embeddings,
            attention_bias=cfg.attention_bias, eos_token_id=cfg.eos_token_ids[0],
            head_dim=cfg.head_dim)
        model = Qwen2ForCausalLM(ref_cfg, tp_size=1).eval()
        load_hf_state_dict(model, tensors)
        ids = token_ids(name, n, cfg.vocab_size)
        backend = NaiveAttentionBackend(ref_cfg)
        meta = AttnMetadata(is_prefill=True, seq_ids=[0], query_lens=[n], context_lens=[n],
                            positions=torch.arange(n, dtype=torch.long))
        with torch.no_grad():
            logits = model.forward_logits_all(torch.tensor(ids, dtype=torch.long), backend, meta)
        np.save(HERE / f"{name}_logits.npy", logits.float().numpy())
        write_safetensors(HERE / f"{name}_weights.safetensors", tensors)
        meta_out[name] = {"tokens": ids, "weights_sha256": checksum(tensors), "seed": SEEDS[name],
                          "torch": torch.__version__}
        print(name, tuple(logits.shape), float(logits.abs().max()))
    (HERE / "golden.json").write_text(json.dumps(meta_out, indent=1) + "\n")


if __name__ == "__main__":
    main()
