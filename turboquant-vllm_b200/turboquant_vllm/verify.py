"""Verify TurboQuant compression quality for a model's cache shape on this GPU.

Mirror of the reference's ``python -m turboquant_vllm.verify`` (reference:
``src/turboquant_vllm/verify.py:124-453``): a 128-token random Gaussian prefill goes through
:class:`turboquant_vllm.CompressedDynamicCache` (here: the sm_100a compress / decompress kernels) and
through a plain ``DynamicCache``; the per-layer cosine similarity of what the two caches hand back
is reported and compared with a threshold (default 0.99).  Same flags, same result keys, same exit
codes (0 PASS, 1 FAIL, 2 bad arguments).

Differences from the reference, both so that the check runs on a machine without the checkpoint:

* only the model's *config* is read (``AutoConfig``), never its weights: the protocol uses nothing of
  the model but its cache shape (layers, KV heads, head dims, layer types);
* ``--model synthetic`` takes the shape from ``--layers / --kv-heads / --head-dim`` instead.

Usage::

    python -m turboquant_vllm.verify --model /path/to/Llama-3.1-8B --bits 4
    python -m turboquant_vllm.verify --model synthetic --layers 32 --kv-heads 8 --head-dim 128 \\
        --k-bits 4 --v-bits 3 --json
"""

from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Any

# config.model_type -> display name of the families the reference lists as validated
# (reference: src/turboquant_vllm/verify.py:49-58)
VALIDATED_MODELS: dict[str, str] = {
    "molmo2": "Molmo2",
    "mistral": "Mistral",
    "llama": "Llama",
    "qwen2": "Qwen2.5",
    "phi3": "Phi",
    "gemma2": "Gemma 2",
    "gemma3": "Gemma 3",
    "gemma4": "Gemma 4",
}

COMPRESSION_QUALITY_THRESHOLD = 0.99  # compressed vs uncompressed, per layer
SEQ_LEN = 128


def _shape_from_config(config: Any) -> dict[str, Any]:
    """Cache shape of a HuggingFace config (reference: ``_detect_model_config``, verify.py:65-121)."""
    text = getattr(config, "text_config", config)
    heads = text.num_attention_heads
    head_dim = getattr(text, "head_dim", None) or text.hidden_size // heads
    return {
        "head_dim": int(head_dim),
        "num_kv_heads": int(getattr(text, "num_key_value_heads", None) or heads),
        "num_layers": int(text.num_hidden_layers),
        "num_kv_shared_layers": int(getattr(text, "num_kv_shared_layers", 0) or 0),
        "global_head_dim": getattr(text, "global_head_dim", None),
        "global_kv_heads": getattr(text, "num_global_key_value_heads", None),
        "layer_types": getattr(text, "layer_types", None),
        "text_config": text,
    }


def _run_verification(
    model_id: str,
    bits: int | None,
    threshold: float,
    *,
    k_bits: int | None = None,
    v_bits: int | None = None,
    synthetic_shape: dict[str, int] | None = None,
    device: str = "cuda:0",
) -> dict[str, Any]:
    """Run the protocol and return the result dict (keys as the reference's, verify.py:306-326).

    Raises:
        ValueError: ``num_kv_shared_layers >= num_hidden_layers`` (no unique cache layer).
        RuntimeError: no CUDA device (the compressed cache has no CPU path).
    """
    import torch
    from transformers import DynamicCache

    from turboquant_vllm.kv_cache import CompressedDynamicCache

    if not torch.cuda.is_available():
        raise RuntimeError("turboquant_vllm.verify needs a CUDA device: the compressed cache runs on the GPU only")

    if synthetic_shape is not None:
        shape = {"head_dim": synthetic_shape["head_dim"], "num_kv_heads": synthetic_shape["kv_heads"],
                 "num_layers": synthetic_shape["layers"], "num_kv_shared_layers": 0, "global_head_dim": None,
                 "global_kv_heads": None, "layer_types": None, "text_config": None}
        validation, family_name = "UNVALIDATED", None
    else:
        from transformers import AutoConfig

        config = AutoConfig.from_pretrained(model_id, trust_remote_code=True, token=os.environ.get("HF_TOKEN"))
        shape = _shape_from_config(config)
        family_name = VALIDATED_MODELS.get(config.model_type)
        validation = "VALIDATED" if family_name else "UNVALIDATED"

    num_cache_layers = shape["num_layers"] - shape["num_kv_shared_layers"]
    if num_cache_layers <= 0:
        raise ValueError(
            f"Model has {shape['num_layers']} layers and {shape['num_kv_shared_layers']} shared KV layers, "
            f"leaving {num_cache_layers} unique cache layers. Check model config for invalid num_kv_shared_layers."
        )
    head_dim, text_config, layer_types = shape["head_dim"], shape["text_config"], shape["layer_types"]

    def make_fake(layer_idx: int, generator: torch.Generator):
        ld, lh = head_dim, shape["num_kv_heads"]
        if layer_types and layer_idx < len(layer_types) and "full" in layer_types[layer_idx]:
            ld = shape["global_head_dim"] or head_dim
            lh = shape["global_kv_heads"] or lh
        dims = (1, lh, SEQ_LEN, ld)
        k = torch.randn(dims, dtype=torch.bfloat16, device=device, generator=generator)
        v = torch.randn(dims, dtype=torch.bfloat16, device=device, generator=generator)
        return k, v

    def new_cache():
        return DynamicCache(config=text_config) if text_config is not None else DynamicCache()

    resolved_k = k_bits if k_bits is not None else bits
    resolved_v = v_bits if v_bits is not None else bits
    per_layer_cosine: list[float] = []
    compressed_cache = new_cache()
    with CompressedDynamicCache(compressed_cache, head_dim=head_dim, bits=bits, k_bits=k_bits, v_bits=v_bits,
                                model_config=text_config):
        rng = torch.Generator(device=device).manual_seed(42)
        for layer_idx in range(num_cache_layers):
            fk, fv = make_fake(layer_idx, rng)
            ck, cv = compressed_cache.update(fk, fv, layer_idx)
            if ck is None or cv is None:
                raise RuntimeError(f"Compressed cache missing keys/values for layer {layer_idx}")
            k_cos = torch.nn.functional.cosine_similarity(fk.flatten().float(), ck.flatten().float(), dim=0).item()
            v_cos = torch.nn.functional.cosine_similarity(fv.flatten().float(), cv.flatten().float(), dim=0).item()
            per_layer_cosine.append(min(k_cos, v_cos))

    min_cosine = min(per_layer_cosine)
    import transformers

    result: dict[str, Any] = {
        "model": model_id,
        "bits": bits if bits is not None else resolved_k,
        "k_bits": resolved_k,
        "v_bits": resolved_v,
        "status": "PASS" if min_cosine >= threshold else "FAIL",
        "validation": validation,
        "threshold": threshold,
        "per_layer_cosine": per_layer_cosine,
        "min_cosine": min_cosine,
        "versions": {"transformers": transformers.__version__, "torch": torch.__version__},
    }
    if family_name is not None:
        result["family_name"] = family_name
    return result


def _format_human_summary(result: dict[str, Any]) -> str:
    """Human-readable summary (reference: verify.py:329-365)."""
    lines = [
        f"Model:      {result['model']}" + (f" ({result['family_name']})" if "family_name" in result else ""),
        f"Bits:       K{result['k_bits']} / V{result['v_bits']}",
        f"Validation: {result['validation']}",
        f"Layers:     {len(result['per_layer_cosine'])}",
        f"Min cosine: {result['min_cosine']:.6f} (threshold {result['threshold']})",
        f"Status:     {result['status']}",
    ]
    if result["validation"] == "UNVALIDATED":
        lines.append("Warning:    this model family is not in the validated list")
    return "\n".join(lines)


def main(argv: list[str] | None = None) -> None:
    """CLI entry point: ``--model``, ``--bits`` or ``--k-bits`` with ``--v-bits``, ``--threshold``,
    ``--json``; exits 0 (PASS) or 1 (FAIL).  Argument rules as the reference's (verify.py:368-449)."""
    parser = argparse.ArgumentParser(description="Verify TurboQuant compression quality on a model's cache shape")
    parser.add_argument("--model", required=True,
                        help="HuggingFace model ID or local directory (only its config is read), or 'synthetic'")
    parser.add_argument("--bits", type=int, choices=[2, 3, 4], default=None,
                        help="Quantization bits per coordinate (shorthand for --k-bits and --v-bits)")
    parser.add_argument("--k-bits", type=int, choices=[2, 3, 4], default=None, help="Key quantization bits")
    parser.add_argument("--v-bits", type=int, choices=[2, 3, 4], default=None, help="Value quantization bits")
    parser.add_argument("--threshold", type=float, default=COMPRESSION_QUALITY_THRESHOLD,
                        help=f"Minimum cosine similarity for PASS (default: {COMPRESSION_QUALITY_THRESHOLD})")
    parser.add_argument("--json", action="store_true", default=False, dest="json_output",
                        help="Output JSON to stdout (human summary to stderr)")
    parser.add_argument("--layers", type=int, default=32, help="--model synthetic: number of layers")
    parser.add_argument("--kv-heads", type=int, default=8, help="--model synthetic: KV heads per layer")
    parser.add_argument("--head-dim", type=int, default=128, help="--model synthetic: head dimension")
    args = parser.parse_args(argv)

    if args.bits is not None and (args.k_bits is not None or args.v_bits is not None):
        parser.error("--bits cannot be used with --k-bits or --v-bits")
    if args.bits is None and args.k_bits is None and args.v_bits is None:
        parser.error("Specify --bits or --k-bits/--v-bits")
    if (args.k_bits is None) != (args.v_bits is None):
        parser.error("--k-bits and --v-bits must be used together")

    synthetic = None
    if args.model == "synthetic":
        synthetic = {"layers": args.layers, "kv_heads": args.kv_heads, "head_dim": args.head_dim}
    result = _run_verification(args.model, args.bits, args.threshold, k_bits=args.k_bits, v_bits=args.v_bits,
                               synthetic_shape=synthetic)
    summary = _format_human_summary(result)
    if args.json_output:
        print(json.dumps(result, indent=2), file=sys.stdout)
        print(summary, file=sys.stderr)
    else:
        print(summary, file=sys.stdout)
    sys.exit(0 if result["status"] == "PASS" else 1)


if __name__ == "__main__":
    main()
