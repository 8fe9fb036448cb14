r"""Baseline vs compressed-cache generation benchmark for a HuggingFace model on this GPU.

Mirror of the reference's ``python -m turboquant_vllm.benchmark`` (reference:
``src/turboquant_vllm/benchmark.py:75-479``) for its ``--compressed`` mode: the same prompt is
generated twice, with a plain ``DynamicCache`` and with every new ``DynamicCache`` wrapped by
:class:`turboquant_vllm.CompressedDynamicCache` (the sm_100a compress / decompress kernels), and the
output texts, peak VRAM, generation time and the cache's compression statistics are reported under
the reference's result keys.

Not built: the reference's default accuracy-only mode (its ``TurboQuantKVCache`` wrapper stores the
lossy tensors uncompressed: a quality probe without a storage path, outside this package's scope)
and video inputs.  ``--compressed`` is therefore implied.

Usage::

    python -m turboquant_vllm.benchmark --model /path/to/Mistral-7B-v0.1 --bits 4 \
        --prompt "The capital of France is" --max-new-tokens 64 --output result.json
"""

from __future__ import annotations

import argparse
import json
import time
from pathlib import Path
from typing import Any

import torch


def _get_vram_mb() -> float:
    return torch.cuda.max_memory_allocated() / (1024 * 1024) if torch.cuda.is_available() else 0.0


def _reset_vram_tracking() -> None:
    if torch.cuda.is_available():
        torch.cuda.reset_peak_memory_stats()
        torch.cuda.empty_cache()


def load_model(model_id: str) -> tuple[Any, Any]:
    """Text model + tokenizer in bfloat16 on the GPU (reference: benchmark.py:75-129, text branch)."""
    from transformers import AutoModelForCausalLM, AutoTokenizer

    tokenizer = AutoTokenizer.from_pretrained(model_id, trust_remote_code=True)
    _reset_vram_tracking()
    model = AutoModelForCausalLM.from_pretrained(model_id, torch_dtype=torch.bfloat16, device_map="cuda",
                                                 trust_remote_code=True)
    return model, tokenizer


def _detect_model_config(model: Any) -> dict[str, int]:
    """Layer / head counts of a loaded model (reference: benchmark.py:204-248)."""
    cfg = getattr(model.config, "text_config", model.config)
    heads = cfg.num_attention_heads
    return {
        "num_layers": int(cfg.num_hidden_layers),
        "num_heads": int(heads),
        "num_kv_heads": int(getattr(cfg, "num_key_value_heads", None) or heads),
        "head_dim": int(getattr(cfg, "head_dim", None) or cfg.hidden_size // heads),
    }


def run_inference(model: Any, tokenizer: Any, prompt: str, max_new_tokens: int = 256) -> tuple[str, float, float]:
    """Greedy generation; returns (new text, peak VRAM MiB, seconds) (reference: benchmark.py:132-201)."""
    enc = tokenizer(prompt, return_tensors="pt")
    input_ids = enc["input_ids"].to(model.device)
    _reset_vram_tracking()
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    t0 = time.perf_counter()
    with torch.no_grad():
        out = model.generate(input_ids, max_new_tokens=max_new_tokens, do_sample=False)
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    elapsed = time.perf_counter() - t0
    text = tokenizer.decode(out[0, input_ids.shape[1]:], skip_special_tokens=True)
    return text, _get_vram_mb(), elapsed


def _patch_cache(cache_cls: type, head_dim: int, bits: int, model_config: Any) -> tuple[Any, list]:
    """Wrap every new ``DynamicCache`` (reference: benchmark.py:251-284).  Returns the original
    ``__init__`` (to restore) and the list that collects the wrappers."""
    from turboquant_vllm.kv_cache import CompressedDynamicCache

    original_init = cache_cls.__init__
    wrappers: list = []

    def patched_init(self_cache: Any, *args: Any, **kwargs: Any) -> None:
        original_init(self_cache, *args, **kwargs)
        wrappers.append(CompressedDynamicCache(self_cache, head_dim=head_dim, bits=bits, model_config=model_config))

    setattr(cache_cls, "__init__", patched_init)  # noqa: B010
    return original_init, wrappers


def run_benchmark(model_id: str, prompt: str, video_path: str | None = None, bits: int = 3,
                  max_new_tokens: int = 256, *, compressed: bool = True, model: Any = None,
                  tokenizer: Any = None) -> dict:
    """Baseline vs compressed-cache comparison (reference: ``run_benchmark``, benchmark.py:287-408).

    ``model`` / ``tokenizer`` may be passed in already loaded (then ``model_id`` is only a label).

    Raises:
        NotImplementedError: ``compressed=False`` or a video input (see the module docstring).
    """
    if not compressed:
        raise NotImplementedError("the accuracy-only mode (TurboQuantKVCache) is not part of this package; "
                                  "pass compressed=True")
    if video_path:
        raise NotImplementedError("video inputs are not supported by this benchmark")
    from transformers import DynamicCache

    if model is None:
        model, tokenizer = load_model(model_id)
    model_cfg = _detect_model_config(model)
    results: dict = {"model_id": model_id, "bits": bits, "mode": "compressed", **model_cfg, "prompt": prompt,
                     "video_path": None}
    base_text, base_vram, base_time = run_inference(model, tokenizer, prompt, max_new_tokens)
    results["baseline"] = {"output_text": base_text, "vram_peak_mib": base_vram, "elapsed_s": base_time}

    text_config = getattr(model.config, "text_config", model.config)
    original_init, wrappers = _patch_cache(DynamicCache, model_cfg["head_dim"], bits, text_config)
    try:
        tq_text, tq_vram, tq_time = run_inference(model, tokenizer, prompt, max_new_tokens)
    finally:
        setattr(DynamicCache, "__init__", original_init)  # noqa: B010
    tq: dict[str, Any] = {"output_text": tq_text, "vram_peak_mib": tq_vram, "elapsed_s": tq_time}
    if wrappers:
        tq["compression_stats"] = wrappers[-1].compression_stats()
    results["turboquant"] = tq
    results["comparison"] = {
        "texts_identical": base_text.strip() == tq_text.strip(),
        "time_ratio": round(tq_time / base_time, 3) if base_time > 0 else 0,
        "vram_delta_mib": round(base_vram - tq_vram, 1),
        "baseline_text_preview": base_text[:200],
        "turboquant_text_preview": tq_text[:200],
    }
    return results


def main(argv: list[str] | None = None) -> None:
    """CLI entry point (flags as the reference's, benchmark.py:411-479)."""
    parser = argparse.ArgumentParser(description="TurboQuant compressed-cache generation benchmark")
    parser.add_argument("--model", required=True, help="HuggingFace model ID or local directory (text model)")
    parser.add_argument("--prompt", default="Describe what you see in detail.", help="Text prompt for inference")
    parser.add_argument("--video", default=None, help="not supported (text-only)")
    parser.add_argument("--bits", type=int, default=3, choices=[2, 3, 4], help="Bits per coordinate")
    parser.add_argument("--max-new-tokens", type=int, default=256, help="Maximum tokens to generate")
    parser.add_argument("--compressed", action="store_true", default=True,
                        help="CompressedDynamicCache (always on: the accuracy-only mode is not built)")
    parser.add_argument("--output", default=None, help="Path to save JSON results (default: stdout)")
    args = parser.parse_args(argv)
    results = run_benchmark(args.model, args.prompt, args.video, args.bits, args.max_new_tokens, compressed=True)
    text = json.dumps(results, indent=2)
    if args.output:
        Path(args.output).write_text(text)
    else:
        print(text)


if __name__ == "__main__":
    main()
