"""The engine at the layer sizes of a real model (hidden 4096, 32 query heads over 8 kv heads of
128, intermediate 12288; two layers and a small vocabulary so that the plain implementation stays
fast): logits under several ways of cutting the work, in 32-bit and in bfloat16."""
import numpy as np
import pytest
import torch

import plain_qwen3 as plain

pytestmark = pytest.mark.gpu

BASE = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=2, head_dim=128, vocab_size=1000,
            max_position_embeddings=4096, rms_norm_eps=1e-6, rope_theta=1000000.0)
CONFIGS = {
    # hidden, heads and intermediate of the 8-billion-parameter shape (untied), of the 4-billion one (tied; query
    # width 4096 over a hidden size of 2560) and of the 32-billion one (64 query heads in groups of 8)
    "8b": dict(BASE, hidden_size=4096, intermediate_size=12288, num_attention_heads=32, num_key_value_heads=8, tie_word_embeddings=False),
    "4b": dict(BASE, hidden_size=2560, intermediate_size=9728, num_attention_heads=32, num_key_value_heads=8, tie_word_embeddings=True),
    "32b": dict(BASE, hidden_size=5120, intermediate_size=25600, num_attention_heads=64, num_key_value_heads=8, tie_word_embeddings=False),
}


@pytest.fixture(scope="module", params=["8b", "4b", "32b"])
def model(request, tmp_path_factory):
    CONFIG = CONFIGS[request.param]
    import kirai_b200  # noqa: F401
    from kirai_b200.registry import config_from_dict
    from kirai_b200.weights import write_random_model

    folder = str(tmp_path_factory.mktemp("real"))
    write_random_model(folder, config_from_dict(CONFIG), seed=2, std=0.02, norm_jitter=0.1)
    config, weights = plain.read_model_folder(folder)
    tokens = torch.randint(0, CONFIG["vocab_size"], (150,), generator=torch.Generator().manual_seed(3)).tolist()
    return dict(folder=folder, tokens=tokens, reference=plain.forward_logits(config, weights, tokens).numpy())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_cuts_at_real_layer_sizes(model, dtype):
    from kirai_b200.engine.batch import StepEntry
    from kirai_b200.engine.runner import ModelRunner

    runner = ModelRunner.from_folder(model["folder"], dtype=dtype, page_size=16, max_tokens=512, num_slots=4)
    tokens, reference = model["tokens"], model["reference"]
    bound = 1e-4 if dtype == "float32" else 0.02 * float(np.abs(reference).max())

    def run(request_id, cuts):
        request = runner.cache.open(request_id)
        rows, start = [], 0
        for count in cuts:
            rows.append(runner.step([StepEntry(request, tokens[start : start + count], range(count))]).cpu().numpy())
            start += count
        runner.cache.close(request)
        return np.concatenate(rows)

    whole = run("whole", [150])
    assert float(np.abs(whole - reference).max()) <= bound
    portions = run("portions", [70, 17, 2, 33, 1, 1, 1, 25])  # crosses the 64-token GEMM variants and page edges
    assert float(np.abs(portions - reference).max()) <= bound
    # two requests side by side: one decodes while the other brings a prompt portion
    a, b = runner.cache.open("a"), runner.cache.open("b")
    first = runner.step([StepEntry(a, tokens[:100], [99])]).cpu().numpy()
    mixed = runner.step([StepEntry(a, tokens[100:101], [0]), StepEntry(b, tokens[:40], range(40))]).cpu().numpy()
    assert float(np.abs(first[0] - reference[99]).max()) <= bound
    assert float(np.abs(mixed[0] - reference[100]).max()) <= bound
    assert float(np.abs(mixed[1:] - reference[:40]).max()) <= bound
    decode = runner.step([StepEntry(a, tokens[101:102], [0]), StepEntry(b, tokens[40:41], [0])]).cpu().numpy()  # decode-only batch
    assert float(np.abs(decode[0] - reference[101]).max()) <= bound
    assert float(np.abs(decode[1] - reference[40]).max()) <= bound
