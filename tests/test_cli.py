"""The `verify` and `benchmark` command-line tools (reference: src/turboquant_vllm/verify.py,
src/turboquant_vllm/benchmark.py; its tests: tests/test_verify.py)."""

from __future__ import annotations

import json

import pytest
import torch

from turboquant_vllm import benchmark, verify


# ---- argument rules (no GPU) -------------------------------------------------------------------------
@pytest.mark.parametrize("argv", [
    ["--model", "synthetic"],                                   # no bit width at all
    ["--model", "synthetic", "--bits", "4", "--k-bits", "4"],   # shorthand mixed with a component flag
    ["--model", "synthetic", "--k-bits", "4"],                  # components only as a pair
    ["--model", "synthetic", "--bits", "7"],                    # outside the supported widths
    ["--bits", "4"],                                            # --model is required
])
def test_verify_rejects_bad_arguments(argv, capsys):
    with pytest.raises(SystemExit) as e:
        verify.main(argv)
    assert e.value.code == 2
    capsys.readouterr()


def test_verify_summary_and_shape_detection():
    class Cfg:
        model_type = "llama"
        num_attention_heads = 32
        num_key_value_heads = 8
        hidden_size = 4096
        num_hidden_layers = 32

    shape = verify._shape_from_config(Cfg())
    assert (shape["head_dim"], shape["num_kv_heads"], shape["num_layers"], shape["num_kv_shared_layers"]) == \
        (128, 8, 32, 0)
    text = verify._format_human_summary({"model": "m", "k_bits": 4, "v_bits": 3, "validation": "UNVALIDATED",
                                         "per_layer_cosine": [0.995, 0.994], "min_cosine": 0.994, "threshold": 0.99,
                                         "status": "PASS"})
    assert "PASS" in text and "K4 / V3" in text and "not in the validated list" in text


def test_benchmark_refuses_the_modes_it_does_not_have():
    with pytest.raises(NotImplementedError):
        benchmark.run_benchmark("m", "p", compressed=False)
    with pytest.raises(NotImplementedError):
        benchmark.run_benchmark("m", "p", video_path="clip.mp4")


# ---- on the GPU ------------------------------------------------------------------------------------------
@pytest.mark.gpu
@pytest.mark.parametrize("bits_args,threshold,code", [
    (["--bits", "4"], "0.99", 0),
    (["--k-bits", "4", "--v-bits", "3"], "0.97", 0),
    (["--bits", "2"], "0.99", 1),   # 2-bit round trips sit near 0.94: FAIL against the default threshold
])
def test_verify_synthetic_shape(bits_args, threshold, code, capsys):
    argv = ["--model", "synthetic", "--layers", "3", "--kv-heads", "8", "--head-dim", "128", "--json",
            "--threshold", threshold, *bits_args]
    with pytest.raises(SystemExit) as e:
        verify.main(argv)
    out = capsys.readouterr()
    result = json.loads(out.out)
    assert e.value.code == code
    assert result["status"] == ("PASS" if code == 0 else "FAIL")
    assert len(result["per_layer_cosine"]) == 3 and result["min_cosine"] == min(result["per_layer_cosine"])
    assert result["validation"] == "UNVALIDATED" and "Status:" in out.err
    if bits_args[0] == "--k-bits":
        assert (result["k_bits"], result["v_bits"]) == (4, 3)
    if code == 0 and bits_args == ["--bits", "4"]:
        assert result["min_cosine"] > 0.994  # 4-bit Lloyd-Max on N(0,1) rows: about 0.9954


class _Tok:
    """Stand-in tokenizer: one token per character code."""

    def __call__(self, text, return_tensors="pt"):
        return {"input_ids": torch.tensor([[3 + (ord(c) % 200) for c in text]], dtype=torch.long)}

    def decode(self, ids, skip_special_tokens=True):
        return " ".join(str(int(i)) for i in ids)


@pytest.mark.gpu
def test_benchmark_on_a_small_random_model():
    """The whole benchmark flow on a 2-layer random Llama: both generations run, every new DynamicCache of
    the second one is wrapped, the statistics describe a 4-bit cache."""
    from transformers import LlamaConfig, LlamaForCausalLM

    torch.manual_seed(0)
    cfg = LlamaConfig(vocab_size=256, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                      num_attention_heads=2, num_key_value_heads=1, head_dim=128, max_position_embeddings=512)
    model = LlamaForCausalLM(cfg).to(device="cuda", dtype=torch.bfloat16).eval()
    res = benchmark.run_benchmark("random-llama", "hello tensor memory", bits=4, max_new_tokens=12,
                                  model=model, tokenizer=_Tok())
    assert res["mode"] == "compressed" and res["num_layers"] == 2 and res["head_dim"] == 128
    assert len(res["baseline"]["output_text"].split()) == 12
    assert len(res["turboquant"]["output_text"].split()) == 12
    stats = res["turboquant"]["compression_stats"]
    assert stats and stats["compression_ratio"] > 3.0
    assert set(res["comparison"]) >= {"texts_identical", "time_ratio", "vram_delta_mib"}
    from transformers import DynamicCache

    assert DynamicCache.__init__.__name__ != "patched_init"  # restored
