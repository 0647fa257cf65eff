"""Each part of a layer alone, and the layer order as data, against the plain functions."""
import math

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
from helpers import TOL

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]
PTOL = {torch.float32: 2e-5, torch.bfloat16: 3e-2}


def rel_err(got, want):
    want = want.to(torch.float64).cpu()
    return float((got.to(torch.float64).cpu() - want).abs().max() / want.abs().max().clamp_min(1e-30))


def weights_for(part, seed=0, gain=1.0):
    """Random tensors (rounded to bfloat16 so that both precisions see the same values) for every
    tensor a part declares; returns (getter, {name: float64 tensor})."""
    g = torch.Generator().manual_seed(seed)
    store = {}
    for s in part.all_tensor_specs():
        if s.init == "norm":
            t = 1 + 0.1 * torch.randn(s.shape, generator=g)
        else:
            t = gain * torch.randn(s.shape, generator=g) / math.sqrt(s.shape[-1])
        store[s.name] = t.to(torch.bfloat16)
    return (lambda n: store[n]), {n: t.double() for n, t in store.items()}


class OnePartModel:
    """The least a runner needs around one block: used to get a step context and a cache."""

    def __init__(self, block, width, dtype):
        from carbon_engine_b200.parts.model import DecoderModel
        from carbon_engine_b200.parts.embedding import Embedding, LMHead
        from carbon_engine_b200.parts.norm import RMSNorm
        emb = Embedding(50, width, "emb")
        self.model = DecoderModel(None, emb, [block], LMHead(50, width, RMSNorm(width, 1e-6, "fn"), None, tied_to=emb))
        get, self.w = weights_for(self.model, seed=1, gain=3.0)
        self.model.load_weights(get, torch.device(DEV), dtype)


def make_runner(model, dtype, page_size=8, pages=64):
    from carbon_engine_b200.cache.storage import CacheStorage
    from carbon_engine_b200.engine.runner import ModelRunner
    storage = CacheStorage(model, dtype, torch.device(DEV), page_size, pages, 4, 256, poison=True)
    return ModelRunner(model, storage, 256)


@pytest.mark.parametrize("dtype", DTYPES)
def test_rmsnorm_part(dtype):
    from carbon_engine_b200.parts.norm import RMSNorm
    n = RMSNorm(80, 3e-6, "x.weight")
    get, w = weights_for(n)
    n.load(get, torch.device(DEV), dtype)
    assert n.weight.dtype == torch.float32                   # held in 32-bit in both precisions
    x = torch.randn(5, 80, device=DEV)
    out = torch.empty(5, 80, dtype=dtype, device=DEV)
    n.forward(x, out)
    assert rel_err(out, plain.rms_norm(x.double().cpu(), w["x.weight"], 3e-6)) < PTOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
def test_linear_part_concatenates_its_tensors(dtype):
    from carbon_engine_b200.parts import linear
    lin = linear.Linear(80, [96, 48, 48], ["q", "k", "v"])
    get, w = weights_for(lin)
    lin.load(get, torch.device(DEV), dtype)
    assert lin.weight.shape == (192, 80) and lin.weight.dtype == dtype
    a = torch.randn(9, 80, device=DEV).to(dtype)
    out = torch.empty(9, 192, dtype=dtype, device=DEV)
    lin.forward(a, out, linear.STORE)
    want = a.double().cpu() @ torch.cat([w["q"], w["k"], w["v"]]).T
    assert rel_err(out, want) < PTOL[dtype]
    x = torch.zeros(9, 192, device=DEV)
    lin.forward(a, x, linear.ACCUM)
    lin.forward(a, x, linear.ACCUM)
    assert rel_err(x, 2 * want) < PTOL[dtype]


def test_rotary_tables():
    from carbon_engine_b200.parts.rope import RotaryEmbedding
    r = RotaryEmbedding(48, 50000.0, 300, rotary_dim=32)
    r.prepare(torch.device(DEV))
    c, s = plain.rope_tables(torch.arange(300), 32, 50000.0)
    assert r.cos.dtype == torch.float32 and r.cos.shape == (300, 16)
    assert torch.equal(r.cos.cpu(), c.float()) and torch.equal(r.sin.cpu(), s.float())


@pytest.mark.parametrize("dtype", DTYPES)
def test_gated_mlp_part(dtype):
    from carbon_engine_b200.parts.mlp import GatedMLP
    from carbon_engine_b200.engine.batch import StepBuffers, StepContext
    mlp = GatedMLP(80, 112, "m")
    get, w = weights_for(mlp, gain=2.0)
    mlp.load_all(get, torch.device(DEV), dtype)
    ctx = StepContext(StepBuffers(16, 2, 0, torch.device(DEV)), 6, 1, dtype, torch.device(DEV), [])
    h = torch.randn(6, 80, device=DEV).to(dtype)
    x = torch.randn(6, 80, device=DEV)
    want = x.double().cpu() + plain.swiglu_mlp(h.double().cpu(), w, "m")
    mlp.forward(ctx, h, x)
    assert rel_err(x, want) < PTOL[dtype]
    with pytest.raises(ValueError, match="silu"):
        GatedMLP(8, 8, "m", activation="gelu")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [0, 21])
def test_attention_part_alone_in_two_steps(dtype, window):
    """The mixer alone: normed activations in, residual out; a prefix in one step, the rest in a
    second step that reads the prefix from the cache."""
    from carbon_engine_b200.parts.attention import PagedAttention
    from carbon_engine_b200.parts.block import PreNormBlock
    from carbon_engine_b200.parts.mlp import GatedMLP
    from carbon_engine_b200.parts.norm import RMSNorm
    from carbon_engine_b200.parts.rope import RotaryEmbedding
    from carbon_engine_b200.engine.batch import StepEntry
    H, nh, nkv, d = 80, 6, 3, 48
    att = PagedAttention(H, nh, nkv, d, "a", RotaryEmbedding(d, 1e4, 256), qk_norm_eps=1e-5, window=window)
    block = PreNormBlock(RMSNorm(H, 1e-5, "n1"), att, RMSNorm(H, 1e-5, "n2"), GatedMLP(H, 112, "m"))
    one = OnePartModel(block, H, dtype)
    runner = make_runner(one.model, dtype)
    runner.open_request(0)
    T, cut = 45, 29
    h = torch.randn(T, H).to(torch.bfloat16)
    cfg = dict(num_attention_heads=nh, num_key_value_heads=nkv, head_dim=d, hidden_size=H, rms_norm_eps=1e-5, rope_theta=1e4)
    want = plain.attention_block(h.double(), one.w, "a", cfg, torch.arange(T), window)
    got = []
    for lo, hi in ((0, cut), (cut, T)):
        ctx, rows, commits = runner.prepare([StepEntry(0, [1] * (hi - lo), [])])
        x = torch.zeros(hi - lo, H, device=DEV)
        att.forward(ctx, h[lo:hi].to(DEV).to(dtype), x, runner.storage.view(one.model.schedule[0]))
        for rid, n in commits:
            runner.storage.manager.commit(rid, n)
        got.append(x)
    runner.check_status()
    assert rel_err(torch.cat(got), want) < PTOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
def test_block_embedding_and_tied_head(dtype):
    from carbon_engine_b200.parts.attention import PagedAttention
    from carbon_engine_b200.parts.block import PreNormBlock
    from carbon_engine_b200.parts.mlp import GatedMLP
    from carbon_engine_b200.parts.norm import RMSNorm
    from carbon_engine_b200.parts.rope import RotaryEmbedding
    from carbon_engine_b200.engine.batch import StepEntry
    H, nh, nkv, d = 64, 4, 2, 16
    att = PagedAttention(H, nh, nkv, d, "model.layers.0.self_attn", RotaryEmbedding(d, 1e4, 256), qk_norm_eps=1e-6)
    block = PreNormBlock(RMSNorm(H, 1e-6, "model.layers.0.input_layernorm.weight"), att,
                         RMSNorm(H, 1e-6, "model.layers.0.post_attention_layernorm.weight"),
                         GatedMLP(H, 96, "model.layers.0.mlp"))
    one = OnePartModel(block, H, dtype)
    m = one.model
    assert m.head.weight.data_ptr() == m.embedding.weight.data_ptr()          # tied: the same memory
    runner = make_runner(m, dtype)
    runner.open_request(0)
    toks = [3, 49, 0, 7, 7, 21, 30, 11, 2]
    ctx, rows, commits = runner.prepare([StepEntry(0, toks, [8, 0])])
    x = torch.empty(len(toks), H, device=DEV)
    m.embedding.forward(ctx, x)
    x_plain = plain.embedding(one.w["emb"], toks)
    assert rel_err(x, x_plain) < 1e-6
    block.forward(ctx, x, runner.storage.view(m.schedule[0]))
    cfg = dict(num_attention_heads=nh, num_key_value_heads=nkv, head_dim=d, hidden_size=H, rms_norm_eps=1e-6, rope_theta=1e4)
    x_plain = plain.decoder_layer(x_plain, one.w, 0, cfg, torch.arange(len(toks)))
    assert rel_err(x, x_plain) < PTOL[dtype]
    logits = m.logits(ctx, x, rows)
    z = plain.rms_norm(x_plain, one.w["fn"], 1e-6) @ one.w["emb"].T
    assert logits.dtype == torch.float32 and rel_err(logits, z[[8, 0]]) < PTOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
def test_layer_order_is_data_a_block_twice_and_a_shared_cache(dtype):
    """Schedule: block 0 (cache 0), block 1 (cache 1), block 0 again (cache 2), block 1 reading cache 1.
    The last call writes no keys: its queries attend to the keys and values its first call stored.
    Block 1's cache has pages of a size of its own, so its page ids and block table are a group apart."""
    from carbon_engine_b200.parts.attention import PagedAttention
    from carbon_engine_b200.parts.block import PreNormBlock
    from carbon_engine_b200.parts.embedding import Embedding, LMHead
    from carbon_engine_b200.parts.mlp import GatedMLP
    from carbon_engine_b200.parts.model import DecoderModel, LayerCall
    from carbon_engine_b200.parts.norm import RMSNorm
    from carbon_engine_b200.parts.rope import RotaryEmbedding
    from carbon_engine_b200.engine.batch import StepEntry
    H, nh, nkv, d, V = 48, 3, 1, 32, 77
    rope = RotaryEmbedding(d, 1e4, 256)
    blocks = [PreNormBlock(RMSNorm(H, 1e-6, f"model.layers.{i}.input_layernorm.weight"),
                           PagedAttention(H, nh, nkv, d, f"model.layers.{i}.self_attn", rope, qk_norm_eps=1e-6,
                                          page_size=4 if i == 1 else None),
                           RMSNorm(H, 1e-6, f"model.layers.{i}.post_attention_layernorm.weight"),
                           GatedMLP(H, 64, f"model.layers.{i}.mlp")) for i in range(2)]
    emb = Embedding(V, H, "model.embed_tokens.weight")
    head = LMHead(V, H, RMSNorm(H, 1e-6, "model.norm.weight"), "lm_head.weight")
    schedule = [LayerCall(0, 0), LayerCall(1, 1), LayerCall(0, 2), LayerCall(1, 1, writes=False)]
    model = DecoderModel(None, emb, blocks, head, schedule)
    assert [c for c, _ in model.cache_layout()] == [0, 1, 2]
    get, w = weights_for(model, seed=3, gain=3.0)
    model.load_weights(get, torch.device(DEV), dtype)
    runner = make_runner(model, dtype)
    assert [g.page_size for g in runner.storage.groups] == [runner.storage.page_size, 4]
    runner.open_request(5)
    toks = np.random.default_rng(0).integers(0, V, 40).tolist()
    got = [runner.step([StepEntry(5, toks[:23], list(range(23)))]), runner.step([StepEntry(5, toks[23:], list(range(17)))])]
    runner.check_status()

    cfg = dict(num_attention_heads=nh, num_key_value_heads=nkv, head_dim=d, hidden_size=H, rms_norm_eps=1e-6,
               rope_theta=1e4, tie_word_embeddings=False)
    pos = torch.arange(40)
    x = plain.embedding(w["model.embed_tokens.weight"], toks)
    x = plain.decoder_layer(x, w, 0, cfg, pos)
    # block 1, first call: remember the keys and values it stores
    p = "model.layers.1"
    h1 = plain.rms_norm(x, w[f"{p}.input_layernorm.weight"], 1e-6)
    cos, sin = plain.rope_tables(pos, d, 1e4)
    k1 = plain.apply_rope(plain.rms_norm((h1 @ w[f"{p}.self_attn.k_proj.weight"].T).view(40, nkv, d),
                                         w[f"{p}.self_attn.k_norm.weight"], 1e-6), cos, sin)
    v1 = (h1 @ w[f"{p}.self_attn.v_proj.weight"].T).view(40, nkv, d)
    x = plain.decoder_layer(x, w, 1, cfg, pos)
    x = plain.decoder_layer(x, w, 0, cfg, pos)
    # block 1 again, reading the stored keys and values with fresh queries
    h = plain.rms_norm(x, w[f"{p}.input_layernorm.weight"], 1e-6)
    q = plain.apply_rope(plain.rms_norm((h @ w[f"{p}.self_attn.q_proj.weight"].T).view(40, nh, d),
                                        w[f"{p}.self_attn.q_norm.weight"], 1e-6), cos, sin)
    a = plain.causal_attention(q, k1, v1, 1 / math.sqrt(d)).reshape(40, nh * d)
    x = x + a @ w[f"{p}.self_attn.o_proj.weight"].T
    x = x + plain.swiglu_mlp(plain.rms_norm(x, w[f"{p}.post_attention_layernorm.weight"], 1e-6), w, f"{p}.mlp")
    want = plain.lm_head(x, w, cfg)
    assert rel_err(torch.cat(got), want) < PTOL[dtype]

    with pytest.raises(ValueError, match="written by two"):
        DecoderModel(None, emb, blocks, head, [LayerCall(0, 0), LayerCall(1, 0)])
    with pytest.raises(ValueError, match="never written"):
        DecoderModel(None, emb, blocks, head, [LayerCall(0, 0), LayerCall(1, 3, writes=False)])
