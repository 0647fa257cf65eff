"""A feed-forward with routing and another position encoding, both defined here, are registered, built,
loaded and stepped without a change to the package.

The toy feed-forward sends every token to the one of E small gated MLPs whose router logit is largest
(router logits in float32) and scales the result by the softmax weight of that logit.  The toy position
encoding rotates the first ``rotary_dim`` elements of a head (fewer than the head has) by angles that
grow linearly with the pair index instead of geometrically.  Neither is a model of anyone's; they only
show that the registries, the loader, the fused q/k kernel (which takes any cos/sin tables) and the
step function take such parts as they are.
"""
from dataclasses import dataclass
from typing import Any, Dict, List

import math
import numpy as np
import pytest
import torch

import plain_qwen3 as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def define_toy():
    from carbon_engine_b200.config.base import ModelConfig
    from carbon_engine_b200.parts.base import FeedForward, TensorSpec, to_device
    from carbon_engine_b200.parts.block import PreNormBlock
    from carbon_engine_b200.parts.embedding import Embedding, LMHead
    from carbon_engine_b200.parts.model import DecoderModel
    from carbon_engine_b200.parts.registry import build_part, register_feed_forward, register_position
    from carbon_engine_b200.parts.rope import PositionEncoding

    class LinearAngles(PositionEncoding):
        """angle(position, i) = position * step * (i + 1), for the first rotary_dim elements of a head; elements
        2i and 2i + 1 turn together (the package's own encoding pairs i with i + rotary_dim / 2)."""
        pairing = "interleaved"

        def __init__(self, head_dim: int, rotary_dim: int, step: float, max_positions: int):
            self.head_dim, self.rotary_dim, self.step, self.max_positions = head_dim, rotary_dim, step, max_positions

        def prepare(self, device) -> None:
            i = torch.arange(1, self.rotary_dim // 2 + 1, dtype=torch.float64)
            ang = torch.arange(self.max_positions, dtype=torch.float64)[:, None] * (self.step * i)[None, :]
            self.cos = ang.cos().to(torch.float32).to(device).contiguous()
            self.sin = ang.sin().to(torch.float32).to(device).contiguous()

    class Top1Experts(FeedForward):
        def __init__(self, hidden: int, intermediate: int, experts: int, prefix: str):
            self.hidden, self.intermediate, self.experts, self.prefix = hidden, intermediate, experts, prefix

        def tensor_specs(self) -> List[TensorSpec]:
            specs = [TensorSpec(f"{self.prefix}.router.weight", (self.experts, self.hidden))]
            for e in range(self.experts):
                specs += [TensorSpec(f"{self.prefix}.experts.{e}.gate_proj.weight", (self.intermediate, self.hidden)),
                          TensorSpec(f"{self.prefix}.experts.{e}.up_proj.weight", (self.intermediate, self.hidden)),
                          TensorSpec(f"{self.prefix}.experts.{e}.down_proj.weight", (self.hidden, self.intermediate))]
            return specs

        def load(self, get, device, dtype) -> None:
            self.router = to_device(get(f"{self.prefix}.router.weight"), device, torch.float32)
            self.w = [[to_device(get(f"{self.prefix}.experts.{e}.{n}_proj.weight"), device, torch.float32)
                       for n in ("gate", "up", "down")] for e in range(self.experts)]

        def forward(self, ctx, h, x) -> None:
            hf = h.float()
            logits = hf @ self.router.T                               # float32
            weight, choice = torch.softmax(logits, dim=-1).max(dim=-1)
            for e in range(self.experts):                             # a token's result depends on that token alone
                rows = (choice == e).nonzero().flatten()
                if rows.numel() == 0:
                    continue
                g, u, d = self.w[e]
                z = hf[rows] @ g.T
                x[rows] += (z * torch.sigmoid(z) * (hf[rows] @ u.T)) @ d.T * weight[rows, None]

    @dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        hidden_size: int = 0
        heads: int = 2
        kv_heads: int = 1
        head_dim: int = 64
        rotary_dim: int = 32
        angle_step: float = 0.05
        experts: int = 3
        expert_width: int = 40
        feed_forwards: tuple = ()

        @classmethod
        def from_dict(cls, raw: Dict[str, Any]) -> "ToyConfig":
            return cls(architecture=raw["architectures"][0], vocab_size=raw["vocab_size"],
                       max_position_embeddings=raw.get("max_position_embeddings", 256), hidden_size=raw["hidden_size"],
                       heads=raw["heads"], kv_heads=raw["kv_heads"], head_dim=raw["head_dim"], rotary_dim=raw["rotary_dim"],
                       angle_step=raw["angle_step"], experts=raw["experts"], expert_width=raw["expert_width"],
                       feed_forwards=tuple(raw["feed_forwards"]))

        def to_json_dict(self) -> Dict[str, Any]:
            return {"architectures": [self.architecture], "vocab_size": self.vocab_size,
                    "max_position_embeddings": self.max_position_embeddings, "hidden_size": self.hidden_size,
                    "heads": self.heads, "kv_heads": self.kv_heads, "head_dim": self.head_dim, "rotary_dim": self.rotary_dim,
                    "angle_step": self.angle_step, "experts": self.experts, "expert_width": self.expert_width,
                    "feed_forwards": list(self.feed_forwards)}

    def build(cfg: ToyConfig, max_positions: int):
        position = build_part("position", "toy_linear_angles", head_dim=cfg.head_dim, rotary_dim=cfg.rotary_dim,
                              step=cfg.angle_step, max_positions=max_positions)
        blocks = []
        for i, kind in enumerate(cfg.feed_forwards):
            p = f"model.layers.{i}"
            if kind == "toy_top1_experts":
                ff = build_part("feed_forward", kind, hidden=cfg.hidden_size, intermediate=cfg.expert_width, experts=cfg.experts,
                                prefix=f"{p}.moe")
            else:
                ff = build_part("feed_forward", kind, hidden=cfg.hidden_size, intermediate=2 * cfg.hidden_size, prefix=f"{p}.mlp")
            mixer = build_part("mixer", "full_attention", hidden=cfg.hidden_size, heads=cfg.heads, kv_heads=cfg.kv_heads,
                               head_dim=cfg.head_dim, prefix=f"{p}.self_attn", position=position, qk_norm_eps=1e-6)
            blocks.append(PreNormBlock(
                build_part("norm", "rmsnorm", width=cfg.hidden_size, eps=1e-6, name=f"{p}.input_layernorm.weight"), mixer,
                build_part("norm", "rmsnorm", width=cfg.hidden_size, eps=1e-6, name=f"{p}.post_attention_layernorm.weight"), ff))
        emb = Embedding(cfg.vocab_size, cfg.hidden_size, "model.embed_tokens.weight")
        head = LMHead(cfg.vocab_size, cfg.hidden_size,
                      build_part("norm", "rmsnorm", width=cfg.hidden_size, eps=1e-6, name="model.norm.weight"), "lm_head.weight")
        return DecoderModel(cfg, emb, blocks, head)

    register_feed_forward("toy_top1_experts", Top1Experts, replace=True)
    register_position("toy_linear_angles", LinearAngles, replace=True)
    return ToyConfig, build


def rotate_interleaved(x, cos, sin):
    """Elements 2i and 2i + 1 of the first 2 * cos.shape[-1] of every head turn by angle i.  x [T, heads, d]."""
    rd = 2 * cos.shape[-1]
    c, s = cos[:, None, :], sin[:, None, :]
    out = x.clone()
    out[..., 0:rd:2] = x[..., 0:rd:2] * c - x[..., 1:rd:2] * s
    out[..., 1:rd:2] = x[..., 1:rd:2] * c + x[..., 0:rd:2] * s
    return out


def plain_toy_forward(cfg: dict, w, tokens):
    """Whole sequence, no cache: the plain functions, with the toy angles and the routing written out."""
    T = len(tokens)
    nh, nkv, d, rd = cfg["heads"], cfg["kv_heads"], cfg["head_dim"], cfg["rotary_dim"]
    i = torch.arange(1, rd // 2 + 1, dtype=torch.float64)
    ang = torch.arange(T, dtype=torch.float64)[:, None] * (cfg["angle_step"] * i)[None, :]
    cos, sin = ang.cos(), ang.sin()
    x = plain.embedding(w["model.embed_tokens.weight"], tokens)
    margin = torch.full((T,), 1.0, dtype=torch.float64)      # smallest gap between a token's two best experts
    for li, kind in enumerate(cfg["feed_forwards"]):
        p = f"model.layers.{li}"
        h = plain.rms_norm(x, w[f"{p}.input_layernorm.weight"], 1e-6)
        q = plain.rms_norm((h @ w[f"{p}.self_attn.q_proj.weight"].T).view(T, nh, d), w[f"{p}.self_attn.q_norm.weight"], 1e-6)
        k = plain.rms_norm((h @ w[f"{p}.self_attn.k_proj.weight"].T).view(T, nkv, d), w[f"{p}.self_attn.k_norm.weight"], 1e-6)
        v = (h @ w[f"{p}.self_attn.v_proj.weight"].T).view(T, nkv, d)
        a = plain.causal_attention(rotate_interleaved(q, cos, sin), rotate_interleaved(k, cos, sin), v, 1.0 / math.sqrt(d))
        x = x + a.reshape(T, nh * d) @ w[f"{p}.self_attn.o_proj.weight"].T
        h = plain.rms_norm(x, w[f"{p}.post_attention_layernorm.weight"], 1e-6)
        if kind == "toy_top1_experts":
            logits = h @ w[f"{p}.moe.router.weight"].T
            probs = torch.softmax(logits, dim=-1)
            weight, choice = probs.max(dim=-1)
            top2 = probs.topk(2, dim=-1).values
            margin = torch.minimum(margin, top2[:, 0] - top2[:, 1])
            out = torch.zeros_like(x)
            for t in range(T):
                e = int(choice[t])
                out[t] = plain.swiglu_mlp(h[t:t + 1], w, f"{p}.moe.experts.{e}")[0] * weight[t]
            x = x + out
        else:
            x = x + plain.swiglu_mlp(h, w, f"{p}.mlp")
    return plain.rms_norm(x, w["model.norm.weight"], 1e-6) @ w["lm_head.weight"].T, margin


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_routed_feed_forward_and_position_encoding(tmp_path, dtype):
    from carbon_engine_b200.cache.storage import CacheStorage
    from carbon_engine_b200.config.registry import load_config, register_architecture, unregister_architecture
    from carbon_engine_b200.engine.batch import StepEntry
    from carbon_engine_b200.engine.engine import build_model, parse_dtype
    from carbon_engine_b200.engine.runner import ModelRunner
    from carbon_engine_b200.parts.registry import unregister_part
    from carbon_engine_b200.weights.loader import write_random_model
    ToyConfig, build = define_toy()
    register_architecture("ToyRoutedForCausalLM", ToyConfig.from_dict, build, replace=True)
    try:
        cfg = ToyConfig(architecture="ToyRoutedForCausalLM", vocab_size=101, max_position_embeddings=256, hidden_size=80,
                        heads=4, kv_heads=2, head_dim=64, rotary_dim=32, angle_step=0.05, experts=3, expert_width=40,
                        feed_forwards=("toy_top1_experts", "gated_mlp", "toy_top1_experts"))
        folder = write_random_model(cfg, str(tmp_path / "toy"), seed=11)
        # decisive routers: the random weights give logits near zero, that is, three nearly equal experts
        import os
        from helpers import read_raw_safetensors, write_safetensors_plain
        path = os.path.join(folder, "model.safetensors")
        raw = read_raw_safetensors(path)
        for n in list(raw):
            if n.endswith("router.weight"):
                raw[n] = raw[n] * 400.0
        write_safetensors_plain(path, raw)
        arch, cfg2 = load_config(folder)
        assert arch.name == "ToyRoutedForCausalLM" and cfg2 == cfg
        model, _, max_len = build_model(folder, parse_dtype(dtype), torch.device(DEV))
        storage = CacheStorage(model, parse_dtype(dtype), torch.device(DEV), 8, 16, 3, max_len, poison=True)
        runner = ModelRunner(model, storage, 128)

        pcfg, w = plain.read_model(folder)
        rng = np.random.default_rng(3)
        seqs = [rng.integers(0, 101, n).tolist() for n in (41, 23)]
        full = [plain_toy_forward(pcfg, w, s) for s in seqs]
        want = [f[0].numpy() for f in full]
        # Routing is a choice, not a sum: where a token's two best experts are nearly tied, 8 bits of mantissa
        # may pick the other one, and everything after that token differs.  In bfloat16 a sequence is
        # therefore compared up to its first token whose gap is below 0.03 (none is dropped in float32).
        if dtype == "float32":
            upto = [len(s) for s in seqs]
        else:
            upto = [int(np.argmax(f[1].numpy() < 0.03)) if (f[1].numpy() < 0.03).any() else len(s) for f, s in zip(full, seqs)]
            assert min(upto) >= 8, "the seed leaves too few comparable tokens: pick another"
        from helpers import TOL, TOL_MODEL_BF16_MEDIAN, TOL_MODEL_BF16_ROW

        def check(got, exp, keep, what):
            if not keep.any():
                return
            err = np.abs(got.cpu().numpy() - exp).max(axis=1)[keep] / np.abs(exp).max()
            if dtype == "float32":
                assert err.max() < TOL["float32"], (what, float(err.max()))
            else:
                assert err.max() < TOL_MODEL_BF16_ROW and np.median(err) < TOL_MODEL_BF16_MEDIAN, (what, float(err.max()))

        runner.open_request(0)
        check(runner.step([StepEntry(0, seqs[0], list(range(41)))]), want[0], np.arange(41) < upto[0], "whole")
        runner.close_request(0)
        # the same sequences in portions, one of them token by token beside the other
        runner.open_request(1); runner.open_request(2)
        p1 = p2 = 0
        sizes = [7, 2, 11, 3, 30]
        k = 0
        while p1 < len(seqs[0]) or p2 < len(seqs[1]):
            entries, exp, keep = [], [], []
            if p1 < len(seqs[0]):
                n = min(sizes[k % len(sizes)], len(seqs[0]) - p1); k += 1
                entries.append(StepEntry(1, seqs[0][p1:p1 + n], list(range(n)))); exp.append(want[0][p1:p1 + n])
                keep.append(np.arange(p1, p1 + n) < upto[0]); p1 += n
            if p2 < len(seqs[1]):
                entries.append(StepEntry(2, seqs[1][p2:p2 + 1], [0])); exp.append(want[1][p2:p2 + 1])
                keep.append(np.arange(p2, p2 + 1) < upto[1]); p2 += 1
            check(runner.step(entries), np.concatenate(exp), np.concatenate(keep), f"mixed at {p1}, {p2}")
        runner.check_status()
        runner.close_request(1); runner.close_request(2)
        storage.manager.check()
    finally:
        unregister_architecture("ToyRoutedForCausalLM")
        unregister_part("feed_forward", "toy_top1_experts")
        unregister_part("position", "toy_linear_angles")
