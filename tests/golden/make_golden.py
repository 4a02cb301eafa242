"""Makes tests/golden/*.pt: logits of ValeGian/liteinfer's own LlamaForCausalLM on tiny random models.

Run once on a CPU, with the reference checkout importable:

    PYTHONPATH=<liteinfer checkout>:<this repo> HF_HUB_OFFLINE=1 python tests/golden/make_golden.py

For each tiny configuration it writes a model folder with this repo's
random-weights mode, loads that folder with the reference's loader
(liteinfer.models.loader.load_hf_model, float32, CPU, "eager" attention), runs
one whole prompt through the reference's own BlockPool / KVCache packed
payload, and stores the prompt, the logits at every position and the
reference's inv_freq.  `tests/test_plain.py` compares `tests/plain_llama.py`
with these files; the model folder is rebuilt there from the same seed.
"""

from __future__ import annotations

import sys
import tempfile
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))

import tiny_configs  # noqa: E402

from liteinfer_b200.weights.random_init import write_random_model  # noqa: E402


def reference_logits(model_dir: Path, tokens: list[int], block_size: int):
    from liteinfer.cache.block_pool import BlockPool
    from liteinfer.cache.kv_cache import KVCache
    from liteinfer.config import EngineConfig
    from liteinfer.models.loader import load_hf_model

    config = EngineConfig(model=str(model_dir), dtype=torch.float32, device="cpu", attn_implementation="eager")
    model, hf = load_hf_model(config, model_dir)
    head_dim = getattr(hf, "head_dim", None) or hf.hidden_size // hf.num_attention_heads
    blocks = -(-len(tokens) // block_size) + 1
    pool = BlockPool(blocks, block_size, hf.num_hidden_layers, hf.num_key_value_heads, head_dim,
                     torch.float32, torch.device("cpu"))
    cache = KVCache(pool)
    cache.reserve(["r"], [len(tokens)])
    payload = cache.make_packed_payload(["r"], [0], [len(tokens)])
    ids = torch.tensor([tokens], dtype=torch.long)
    positions = torch.arange(len(tokens), dtype=torch.long)[None, :]
    with torch.no_grad():
        out = model(input_ids=ids, position_ids=positions, past_key_values=payload, logits_positions=None)
    return out.logits[0].float(), model.model.rotary_emb.inv_freq.float().clone()


def main() -> None:
    for name, (config, seed, page) in tiny_configs.ALL.items():
        tokens = tiny_configs.prompt(config["vocab_size"], 45, seed)
        with tempfile.TemporaryDirectory() as tmp:
            model_dir = write_random_model(config, Path(tmp) / name, seed, dtype=torch.float32)
            logits, inv_freq = reference_logits(model_dir, tokens, page)
        torch.save({"tokens": tokens, "logits": logits, "inv_freq": inv_freq, "seed": seed},
                   HERE / f"{name}.pt")
        print(name, tuple(logits.shape), float(logits.abs().max()))


if __name__ == "__main__":
    main()
