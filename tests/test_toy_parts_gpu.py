"""A mixer with state of its own, defined here, is registered, built, loaded and stepped without a
change to the package: the parts registry, the architecture registry, the random-weights writer,
the loader, the cache manager's state slots and the step function all take it as it is.

The toy model alternates attention layers with layers whose mixer is a decaying sum over the
sequence: s_t = decay * s_{t-1} + W_in h_t, out_t = W_out s_t, with s kept per request in a state
slot between steps.  It is no model of anyone's; it only shows the interfaces.
"""
from dataclasses import dataclass
from typing import Any, Dict, List

import numpy as np
import pytest
import torch

import plain_qwen3 as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def define_toy():
    from carbon_engine_b200.config.base import ModelConfig
    from carbon_engine_b200.parts.base import Mixer, StateCacheSpec, TensorSpec, to_device
    from carbon_engine_b200.parts.block import PreNormBlock
    from carbon_engine_b200.parts.embedding import Embedding, LMHead
    from carbon_engine_b200.parts.model import DecoderModel
    from carbon_engine_b200.parts.registry import build_part, register_mixer

    class DecayMixer(Mixer):
        def __init__(self, hidden: int, state: int, decay: float, prefix: str):
            self.hidden, self.state_width, self.decay, self.prefix = hidden, state, decay, prefix

        def tensor_specs(self) -> List[TensorSpec]:
            return [TensorSpec(f"{self.prefix}.in.weight", (self.state_width, self.hidden)),
                    TensorSpec(f"{self.prefix}.out.weight", (self.hidden, self.state_width))]

        def load(self, get, device, dtype) -> None:
            self.w_in = to_device(get(f"{self.prefix}.in.weight"), device, torch.float32)
            self.w_out = to_device(get(f"{self.prefix}.out.weight"), device, torch.float32)

        def cache_spec(self):
            return StateCacheSpec((self.state_width,), torch.float32)

        def forward(self, ctx, h, x, cache) -> None:
            u = h.float() @ self.w_in.T                              # [T, state]
            for b in range(ctx.B):                                   # a state mixer takes each sequence's tokens in order
                lo, hi = ctx.h_q_start[b], ctx.h_q_start[b + 1]
                s = cache.state[ctx.h_slots[b]]
                if ctx.h_ctx_before[b] == 0:
                    s.zero_()
                for t in range(lo, hi):
                    s.mul_(self.decay).add_(u[t])
                    x[t] += s @ self.w_out.T

    @dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        hidden_size: int = 0
        state_size: int = 0
        decay: float = 0.9
        mixers: tuple = ()
        heads: int = 2
        head_dim: int = 16

        @classmethod
        def from_dict(cls, raw: Dict[str, Any]) -> "ToyConfig":
            return cls(architecture=raw["architectures"][0], vocab_size=raw["vocab_size"],
                       max_position_embeddings=raw.get("max_position_embeddings", 256), hidden_size=raw["hidden_size"],
                       state_size=raw["state_size"], decay=raw["decay"], mixers=tuple(raw["mixers"]),
                       heads=raw["heads"], head_dim=raw["head_dim"])

        def to_json_dict(self) -> Dict[str, Any]:
            return {"architectures": [self.architecture], "vocab_size": self.vocab_size,
                    "max_position_embeddings": self.max_position_embeddings, "hidden_size": self.hidden_size,
                    "state_size": self.state_size, "decay": self.decay, "mixers": list(self.mixers),
                    "heads": self.heads, "head_dim": self.head_dim}

    def build(cfg: ToyConfig, max_positions: int):
        rope = build_part("position", "rotary", head_dim=cfg.head_dim, theta=1e4, max_positions=max_positions)
        blocks = []
        for i, kind in enumerate(cfg.mixers):
            p = f"model.layers.{i}"
            if kind == "toy_decay":
                mixer = build_part("mixer", kind, hidden=cfg.hidden_size, state=cfg.state_size, decay=cfg.decay, prefix=f"{p}.mix")
            else:
                mixer = build_part("mixer", kind, hidden=cfg.hidden_size, heads=cfg.heads, kv_heads=1, head_dim=cfg.head_dim,
                                   prefix=f"{p}.self_attn", position=rope, qk_norm_eps=1e-6)
            blocks.append(PreNormBlock(
                build_part("norm", "rmsnorm", width=cfg.hidden_size, eps=1e-6, name=f"{p}.input_layernorm.weight"), mixer,
                build_part("norm", "rmsnorm", width=cfg.hidden_size, eps=1e-6, name=f"{p}.post_attention_layernorm.weight"),
                build_part("feed_forward", "gated_mlp", hidden=cfg.hidden_size, intermediate=2 * cfg.hidden_size, prefix=f"{p}.mlp")))
        emb = Embedding(cfg.vocab_size, cfg.hidden_size, "model.embed_tokens.weight")
        head = LMHead(cfg.vocab_size, cfg.hidden_size,
                      build_part("norm", "rmsnorm", width=cfg.hidden_size, eps=1e-6, name="model.norm.weight"), "lm_head.weight")
        return DecoderModel(cfg, emb, blocks, head)

    register_mixer("toy_decay", DecayMixer, replace=True)
    return ToyConfig, build


def plain_toy_forward(cfg: dict, w, tokens):
    """Whole sequence, no cache, from the plain functions plus the recurrence written out."""
    T = len(tokens)
    pos = torch.arange(T)
    x = plain.embedding(w["model.embed_tokens.weight"], tokens)
    acfg = dict(num_attention_heads=cfg["heads"], num_key_value_heads=1, head_dim=cfg["head_dim"],
                hidden_size=cfg["hidden_size"], rms_norm_eps=1e-6, rope_theta=1e4)
    for i, kind in enumerate(cfg["mixers"]):
        p = f"model.layers.{i}"
        h = plain.rms_norm(x, w[f"{p}.input_layernorm.weight"], 1e-6)
        if kind == "toy_decay":
            u = h @ w[f"{p}.mix.in.weight"].T
            s = torch.zeros(cfg["state_size"], dtype=torch.float64)
            out = []
            for t in range(T):
                s = cfg["decay"] * s + u[t]
                out.append(s @ w[f"{p}.mix.out.weight"].T)
            x = x + torch.stack(out)
        else:
            x = x + plain.attention_block(h, w, f"{p}.self_attn", acfg, pos)
        x = x + plain.swiglu_mlp(plain.rms_norm(x, w[f"{p}.post_attention_layernorm.weight"], 1e-6), w, f"{p}.mlp")
    return plain.rms_norm(x, w["model.norm.weight"], 1e-6) @ w["lm_head.weight"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_state_mixer_is_registered_built_and_stepped(tmp_path, dtype):
    from carbon_engine_b200.cache.storage import CacheStorage
    from carbon_engine_b200.config.registry import load_config, register_architecture, unregister_architecture
    from carbon_engine_b200.engine.batch import StepEntry
    from carbon_engine_b200.engine.engine import build_model, parse_dtype
    from carbon_engine_b200.engine.runner import ModelRunner
    from carbon_engine_b200.parts.base import StateCacheSpec
    from carbon_engine_b200.parts.registry import unregister_part
    from carbon_engine_b200.weights.loader import write_random_model
    ToyConfig, build = define_toy()
    register_architecture("ToyDecayForCausalLM", ToyConfig.from_dict, build, replace=True)
    try:
        cfg = ToyConfig(architecture="ToyDecayForCausalLM", vocab_size=90, max_position_embeddings=256, hidden_size=48,
                        state_size=24, decay=0.8, mixers=("full_attention", "toy_decay", "toy_decay", "full_attention"),
                        heads=3, head_dim=16)
        folder = write_random_model(cfg, str(tmp_path / "toy"), seed=4)
        arch, cfg2 = load_config(folder)
        assert arch.name == "ToyDecayForCausalLM" and cfg2 == cfg
        model, _, max_len = build_model(folder, parse_dtype(dtype), torch.device(DEV))
        kinds = [type(s).__name__ for _, s in model.cache_layout()]
        assert kinds == ["PagedCacheSpec", "StateCacheSpec", "StateCacheSpec", "PagedCacheSpec"]
        storage = CacheStorage(model, parse_dtype(dtype), torch.device(DEV), 8, 24, 3, max_len, poison=True)
        assert len(storage.groups) == 1                      # the two attention layers share one group of pages
        runner = ModelRunner(model, storage, 128)

        pcfg, w = plain.read_model(folder)
        rng = np.random.default_rng(8)
        seqs = [rng.integers(0, 90, n).tolist() for n in (37, 20, 51)]
        want = [plain_toy_forward(pcfg, w, s).numpy() for s in seqs]
        tol = 1e-4 if dtype == "float32" else 3e-2

        def check(got, exp, what):
            err = np.abs(got.cpu().numpy() - exp).max() / np.abs(exp).max()
            assert err < tol, (what, err)

        # whole
        runner.open_request(0)
        check(runner.step([StepEntry(0, seqs[0], list(range(37)))]), want[0], "whole")
        runner.close_request(0)
        # in portions, two requests side by side, one of them token by token; the state slot of request 0 is reused
        runner.open_request(1); runner.open_request(2)
        p1 = p2 = 0
        sizes = [5, 2, 9, 3, 30]
        k = 0
        while p1 < len(seqs[1]) or p2 < len(seqs[2]):
            entries, exp = [], []
            if p1 < len(seqs[1]):
                entries.append(StepEntry(1, seqs[1][p1:p1 + 1], [0])); exp.append(want[1][p1:p1 + 1]); p1 += 1
            if p2 < len(seqs[2]):
                n = min(sizes[k % len(sizes)], len(seqs[2]) - p2); k += 1
                entries.append(StepEntry(2, seqs[2][p2:p2 + n], list(range(n)))); exp.append(want[2][p2:p2 + n]); p2 += n
            check(runner.step(entries), np.concatenate(exp), f"mixed at {p1}, {p2}")
        runner.check_status()
        runner.close_request(1); runner.close_request(2)
        storage.manager.check()
        assert storage.manager.free_pages(0) == 24 and storage.manager.free_slots() == 3
        # through the entry point: the per-request state is part of the memory the cache is sized beside
        from carbon_engine_b200 import Engine, SamplingParams
        eng = Engine(folder, dtype=dtype, page_size=8, max_running_requests=3, max_prefill_tokens=64, memory_ratio=0.3)
        assert eng._state_bytes() == 2 * 24 * 4 * 3 == eng.storage.state_bytes()       # two state layers, float32, 3 slots
        assert eng._workspace_bytes() > eng.model.step_bytes(64, 4, rows=3) > 0
        assert not eng.cuda_graphs and eng.stats()["kv_pages_total"] == 8 * max_len // 8
        out = eng.generate([seqs[1]], SamplingParams(max_tokens=4, ignore_eos=True))[0]
        toks = list(seqs[1])
        for t in out.token_ids:
            row = plain_toy_forward(pcfg, w, toks)[-1]
            assert t == int(row.argmax()) or float(row.max() - row[t]) < 2 * tol * float(row.abs().max())
            toks.append(t)
    finally:
        unregister_architecture("ToyDecayForCausalLM")
        unregister_part("mixer", "toy_decay")
