"""Writes tests/golden/*.npz: logits of the reference's own model code on tiny random models.

Run from the repository root on a machine that has the reference checkout (path in
``VELOX_REFERENCE``, a read-only source tree) and no GPU:

    TRITON_INTERPRET=1 VELOX_REFERENCE=<path> python tests/golden/make_golden.py

The reference's Triton kernels run on the CPU under the Triton interpreter, in float32.  The
model folders are written by this repository's random-weights mode and read by the reference's
own loader, so the run also shows that the tensor names and the q,k,v / gate,up order agree.
Logits at every position are obtained the way the reference's tests do it
(tests/test_engine_e2e.py:107-124): schedule the request, then call the runner's
``prepare_prefill``/``prepare_decode``, ``forward`` and ``compute_logits`` by hand.  Each prompt
is fed in portions (so the reference's paged prefill kernel runs with context) and its last
token alone (so the decode kernel runs too).
"""
import json
import os
import sys
import tempfile

os.environ.setdefault("TRITON_INTERPRET", "1")
os.environ.setdefault("HF_HUB_OFFLINE", "1")

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
REFERENCE = os.environ.get("VELOX_REFERENCE", "")
if not os.path.isdir(REFERENCE):
    sys.exit("set VELOX_REFERENCE to the reference checkout")
sys.path.insert(0, REFERENCE)
sys.path.insert(1, ROOT)
sys.path.insert(2, os.path.join(ROOT, "tests"))

import numpy as np  # noqa: E402
import torch  # noqa: E402

from engine.config import EngineConfig  # noqa: E402  (reference)
from engine.engine import Engine  # noqa: E402  (reference)
from src.config import ModelConfig  # noqa: E402  (reference)
from src.paged_kv_cache import PagedKVCache  # noqa: E402  (reference)
from src.transformer import QwenForCausalLM  # noqa: E402  (reference)
from src.weight_loader import load_qwen_weights  # noqa: E402  (reference)
from engine.request import Request  # noqa: E402  (reference)
from engine.utils import SamplingParams  # noqa: E402  (reference)

import tiny_configs  # noqa: E402
from velox_b200.weights import write_random_model  # noqa: E402

CASES = {
    # name: (config, weights seed, page size, portion size, prompt lengths, prompt seed)
    "tiny_a": (tiny_configs.TINY_A, 11, 4, 4, (5, 11, 17), 101),
    "tiny_b": (tiny_configs.TINY_B, 12, 8, 16, (1, 9, 33, 70), 102),
}


def reference_config(folder, cfg):
    """The reference's ``ModelConfig`` from the config.json keys, through its public constructor.

    Its ``from_hf`` goes through ``transformers.AutoConfig.to_dict()``, and the transformers
    version installed here moves ``rope_theta`` into a nested ``rope_parameters`` entry, so
    ``from_hf`` would fall back to its default of 10000 (src/config.py:39) whatever config.json
    says.  Building the dataclass from the same keys with the same defaults (src/config.py:29-42)
    keeps the run on the reference's model code and off that version mismatch.
    """
    heads = int(cfg["num_attention_heads"])
    return ModelConfig(
        model_name=folder,
        hidden_size=int(cfg["hidden_size"]),
        num_hidden_layers=int(cfg["num_hidden_layers"]),
        num_attention_heads=heads,
        num_key_value_heads=int(cfg.get("num_key_value_heads", heads)),
        intermediate_size=int(cfg["intermediate_size"]),
        rms_norm_eps=float(cfg.get("rms_norm_eps", 1e-6)),
        vocab_size=int(cfg["vocab_size"]),
        max_position_embeddings=int(cfg.get("max_position_embeddings", 4096)),
        rope_theta=float(cfg.get("rope_theta", 10000.0)),
        rope_scaling=cfg.get("rope_scaling"),
        tie_word_embeddings=bool(cfg.get("tie_word_embeddings", False)),
    )


def all_position_logits(engine, token_ids, name):
    request = Request(name, list(token_ids), SamplingParams(temperature=0.0, max_tokens=2, ignore_eos=True))
    engine.scheduler.add_request(request)
    rows = []
    with torch.no_grad():
        while request.num_computed_tokens < len(token_ids):
            out = engine.scheduler.schedule()
            if out.prefill_batch:
                assert out.prefill_batch == [request]
                ids, meta = engine.runner.prepare_prefill([request])
            else:
                assert out.decode_batch == [request]
                ids, meta = engine.runner.prepare_decode([request])
                meta.num_splits = 1
            hidden = engine.runner.forward(ids, meta)
            rows.append(engine.model.compute_logits(hidden).float())
            request.num_computed_tokens += request.current_chunk_size
            request.refresh_status()
    engine.scheduler.abort_request(name)
    return torch.cat(rows)


def main():
    out_dir = os.path.dirname(os.path.abspath(__file__))
    for case, (cfg, wseed, page, portion, lengths, pseed) in CASES.items():
        with tempfile.TemporaryDirectory() as folder:
            write_random_model(folder, cfg, seed=wseed, dtype="float32")
            model_config = reference_config(folder, cfg)
            model = QwenForCausalLM(model_config, max_position=cfg["max_position_embeddings"]).float()
            load_qwen_weights(model, model_config, folder)
            model.eval()
            heads = cfg["num_attention_heads"]
            cache = PagedKVCache(
                cfg["num_hidden_layers"], cfg["num_key_value_heads"], cfg["hidden_size"] // heads,
                num_blocks=40, block_size=page, dtype=torch.float32, device="cpu", verbose=False,
            )
            engine = Engine(
                model,
                cache,
                EngineConfig(
                    model=folder, dtype="float32", device="cpu", max_model_len=cfg["max_position_embeddings"],
                    max_num_seqs=4, max_num_batched_tokens=64, max_prefill_chunk_size=portion,
                    block_size=page, num_gpu_blocks=40, enable_prefix_caching=False, enable_cuda_graphs=False,
                ),
                eos_token_ids=[],
            )
        gen = torch.Generator().manual_seed(pseed)
        arrays = {"weights_seed": np.int64(wseed)}
        for index, length in enumerate(lengths):
            ids = torch.randint(0, cfg["vocab_size"], (length,), generator=gen).tolist()
            logits = all_position_logits(engine, ids, f"g{index}")
            arrays[f"ids_{index}"] = np.asarray(ids, dtype=np.int32)
            arrays[f"logits_{index}"] = logits.numpy().astype(np.float32)
            print(case, "prompt", index, "len", length, "logits", tuple(logits.shape))
        np.savez_compressed(os.path.join(out_dir, f"{case}.npz"), **arrays)
    print("wrote", sorted(f for f in os.listdir(out_dir) if f.endswith(".npz")))


if __name__ == "__main__":
    main()
