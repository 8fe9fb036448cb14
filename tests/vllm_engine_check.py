"""Engine-level check of the plugin: a tiny random-weight Llama (2 layers, 8 q / 2 kv heads,
head_dim 128) served by vLLM with ``--attention-backend CUSTOM`` (this package's TQ4 backend) and
with vLLM's default backend; greedy generations of the same prompts must agree token for token
(TQ4 is near-lossless at this scale).  Not collected by pytest (engine start-up takes a minute per
backend); run it by hand on a GPU box:

    python tests/vllm_engine_check.py            # CUSTOM with CUDA graphs, then the default backend
    python tests/vllm_engine_check.py CUSTOM eager
"""

from __future__ import annotations

import json
import os
import subprocess
import sys
import tempfile

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CONFIG = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_size": 1024,
    "intermediate_size": 2048, "num_hidden_layers": 2, "num_attention_heads": 8,
    "num_key_value_heads": 2, "head_dim": 128, "vocab_size": 2048, "max_position_embeddings": 4096,
    "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "hidden_act": "silu", "tie_word_embeddings": False,
    "torch_dtype": "bfloat16", "bos_token_id": 1, "eos_token_id": 2,
}


def run_engine(backend: str, eager: bool, model_dir: str) -> list[list[int]]:
    """Generate 24 greedy tokens for four seeded prompts; returns the token ids."""
    sys.path[:0] = [os.path.join(ROOT, "turboquant-vllm_b200")]
    os.environ.setdefault("VLLM_ENABLE_V1_MULTIPROCESSING", "0")
    import torch

    if backend == "CUSTOM":
        from turboquant_vllm.vllm import register_tq4_backend

        register_tq4_backend()
    from vllm import LLM, SamplingParams

    kw = {"attention_config": {"backend": backend}} if backend != "DEFAULT" else {}
    llm = LLM(model=model_dir, load_format="dummy", skip_tokenizer_init=True, enforce_eager=eager,
              max_model_len=2048, gpu_memory_utilization=0.25, seed=0, dtype="bfloat16", **kw)
    g = torch.Generator().manual_seed(0)
    prompts = [{"prompt_token_ids": torch.randint(3, 2000, (n,), generator=g).tolist()} for n in (40, 300, 7, 129)]
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=24, detokenize=False))
    return [list(o.outputs[0].token_ids) for o in outs]


def main() -> int:
    if len(sys.argv) >= 3:  # child: one backend, print the tokens as JSON on the last line
        backend, mode, model_dir = sys.argv[1], sys.argv[2], sys.argv[3]
        print("TOKENS " + json.dumps(run_engine(backend, mode == "eager", model_dir)))
        return 0
    with tempfile.TemporaryDirectory() as d:
        with open(os.path.join(d, "config.json"), "w") as f:
            json.dump(CONFIG, f)
        results = {}
        for backend, mode in (("CUSTOM", "graphs"), ("DEFAULT", "eager")):
            out = subprocess.run([sys.executable, os.path.abspath(__file__), backend, mode, d],
                                 capture_output=True, text=True, timeout=900)
            lines = [ln for ln in out.stdout.splitlines() if ln.startswith("TOKENS ")]
            if not lines:
                print(out.stdout[-2000:], out.stderr[-2000:])
                return 1
            results[backend] = json.loads(lines[-1][7:])
        same = results["CUSTOM"] == results["DEFAULT"]
        print("CUSTOM (TQ4, CUDA graphs) vs default backend:", "identical tokens" if same else "DIFFERENT")
        for a, b in zip(results["CUSTOM"], results["DEFAULT"]):
            print(a[:12], b[:12])
        return 0 if same else 2


if __name__ == "__main__":
    sys.exit(main())
