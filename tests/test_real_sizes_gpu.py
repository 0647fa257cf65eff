"""Two layers at the TRUE layer sizes of the model the benchmark runs (width 4096, 32 query heads on 8
KV heads of 128, intermediate 12288, vocabulary 151936, untied head), in float32 and bfloat16, against
the plain implementation run on the GPU in float64.

One prompt of 300 tokens is run whole and, as a second request, as 200 + 68 tokens followed by its last
32 tokens one by one, with a cache so small that the second request gets the first one's pages.  At
these sizes the bfloat16 steps run the kernels the benchmark times: the CTA-pair tcgen05 product and
the tcgen05 flash kernel (300 and 200 tokens), split-K products whose splits add together (68 tokens),
and the split-K products and the TMA decode kernel with its merge inside a cluster (one token).  The
reference checks its fused attention at a real head geometry in its self-test
(src/device.rs:776-848, 963-1023) and runs its equivalence suite on the serving device
(tests/parallel.rs:104-126).

The q/k norm weights are scaled as in the tiny test models (scores twice as large), so that attention is
peaked and a misplaced key moves the logits; much larger scores would lose absolute precision in
bfloat16 keys and queries.
"""
import numpy as np
import pytest
import torch

import plain_qwen3 as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

SIZES = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=2, hidden_size=4096,
             num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=12288, vocab_size=151936,
             rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=40960)
SHARPEN = 2.0


@pytest.fixture(scope="module")
def material():
    """(typed config, plain config, float64 weights on the GPU, prompt, plain logits of the whole prompt)."""
    import carbon_engine_b200.models  # noqa: F401
    from carbon_engine_b200.config.qwen3 import Qwen3Config
    from carbon_engine_b200.config.registry import resolve_architecture
    from carbon_engine_b200.weights.random_init import RandomWeights
    cfg = Qwen3Config.from_dict(dict(SIZES))
    model = resolve_architecture(cfg.to_json_dict()).build_model(cfg, 1024)
    gen = RandomWeights(model.all_tensor_specs(), 7, torch.device(DEV))
    w = {}
    for spec in model.all_tensor_specs():
        t = gen(spec.name).to(torch.float64)
        if spec.name.endswith(("q_norm.weight", "k_norm.weight")):
            t = t * SHARPEN ** 0.5
        w[spec.name] = t
    prompt = np.random.default_rng(17).integers(0, SIZES["vocab_size"], 300).tolist()
    with torch.no_grad():
        want = plain.forward(dict(SIZES), w, prompt)
    del w["model.embed_tokens.weight"], w["lm_head.weight"]          # 10 GB in float64: not needed again
    return cfg, prompt, want


def make_runner(cfg, dtype):
    from carbon_engine_b200.cache.storage import CacheStorage
    from carbon_engine_b200.engine.engine import build_model
    from carbon_engine_b200.engine.runner import ModelRunner
    model, _, _ = build_model(None, dtype, torch.device(DEV), config=cfg, dummy_weight=True, seed=7, max_seq_len=1024)
    for block in model.blocks:
        block.mixer.q_norm_weight *= SHARPEN ** 0.5
        block.mixer.k_norm_weight *= SHARPEN ** 0.5
    # 6 pages of 64: the prompt needs 5, so the second request reuses the pages of the first
    storage = CacheStorage(model, dtype, torch.device(DEV), 64, 6, 2, 1024, poison=True)
    return ModelRunner(model, storage, 512)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_two_layers_of_the_benchmarks_sizes_whole_and_cut(material, dtype):
    from carbon_engine_b200 import ops
    from carbon_engine_b200.engine.batch import StepEntry
    cfg, prompt, want = material
    runner = make_runner(cfg, dtype)
    ops.reset_kernel_counts()
    tol = 1e-4 if dtype == torch.float32 else 3e-2
    scale = float(want.abs().max())

    def err(got, rows):
        return float((got.double() - want[rows]).abs().max()) / scale

    runner.open_request(0)
    whole = runner.step([StepEntry(0, prompt, list(range(300)))]).clone()
    runner.check_status()
    runner.close_request(0)
    assert torch.isfinite(whole).all()
    assert err(whole, slice(0, 300)) < tol
    # the same prompt again in pieces, over the pages the first request gave back
    runner.open_request(1)
    got = [runner.step([StepEntry(1, prompt[:200], list(range(200)))]).clone(),
           runner.step([StepEntry(1, prompt[200:268], list(range(68)))]).clone()]
    for p in range(268, 300):
        got.append(runner.step([StepEntry(1, [prompt[p]], [0])]).clone())
    runner.check_status()
    runner.close_request(1)
    runner.storage.manager.check()
    cut = torch.cat(got)
    assert torch.isfinite(cut).all()
    assert err(cut, slice(0, 300)) < tol
    if dtype == torch.float32:
        assert torch.equal(cut, whole)                    # 32-bit: the cut changes no bit
    else:
        # greedy picks agree with the plain implementation wherever it has a clear winner
        top2 = want.topk(2, dim=-1).values
        clear = (top2[:, 0] - top2[:, 1]) > 2 * tol * scale
        assert int(clear.sum()) > 30                     # (152 K candidates: the two best are often close)
        assert torch.equal(cut.argmax(-1)[clear], want.argmax(-1)[clear])
        launched = ops.kernel_counts()
        for name in ("gemm_tc_pair_kernel", "attention_prefill_tc_kernel", "attention_decode_tma_kernel (merge in the cluster)",
                     "gemm_tc_kernel (split-K)", "gemm_tc_kernel (split-K, splits add together)"):
            assert launched.get(name, 0) > 0, (name, sorted(launched))
