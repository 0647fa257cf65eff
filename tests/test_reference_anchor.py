"""The plain implementation against output of pedrosoares/carbon-engine's OWN code.

The reference's model code (Rust on a tensor library) cannot be built where these tests run, but four
of its CUDA kernel sources compile as plain C++ with the CUDA keywords defined away
(tests/golden/reference_kernels_host.cpp).  tests/golden/reference_vectors.npz holds seeded inputs and
what those sources computed for them (made by tests/golden/make_reference_vectors.py).  Pinned by that
output, at 1e-5:

* ``plain.causal_attention``: grouped heads, scale, the causal offset of new queries over a cached
  prefix, slot tables (src/kernels/attention.cu ``paged_decode_f32``, ``flash_prefill_f32``);
* ``plain.rms_norm`` followed by ``plain.apply_rope`` with a partial rotary width
  (src/kernels/qsa.cu:98-116, inside ``qsa_select_f32``);
* the sampler's uniforms, ``sampling.sampler.mix64`` and the formula the GPU sampler's tests use
  (src/kernels/sampling.cu:30-42 ``carbon_uniform``).

SwiGLU, the order of operations in a layer and the head still rest on reading the reference's formulas.
With CARBON_REFERENCE_ROOT pointing at a checkout of the reference (and g++ at hand) the vectors are
made afresh and must equal the committed ones.
"""
import math
import os
import shutil
import sys

import numpy as np
import pytest
import torch

import plain_qwen3 as plain

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.fixture(scope="module")
def vec():
    return dict(np.load(os.path.join(GOLDEN, "reference_vectors.npz")))


def _rel(got, want):
    return float(np.abs(np.asarray(got, dtype=np.float64) - want).max() / np.abs(want).max())


def test_decode_attention_matches_the_reference_kernel(vec):
    B, H, KVH, D = (int(v) for v in vec["decode_dims"])
    scale = float(vec["decode_scale"][0])
    k, v, slots, starts = vec["decode_k"], vec["decode_v"], vec["decode_slots"], vec["decode_starts"]
    for b in range(B):
        own = slots[starts[b]:starts[b + 1]].astype(np.int64)          # the sequence's positions, in order
        L = len(own)
        q_all = torch.zeros(L, H, D, dtype=torch.float64)
        q_all[L - 1] = torch.from_numpy(vec["decode_q"][b]).double()
        got = plain.causal_attention(q_all, torch.from_numpy(k[own]).double(), torch.from_numpy(v[own]).double(), scale)[L - 1]
        assert _rel(got.numpy(), vec["decode_out"][b]) < 1e-5, b


def test_prefill_attention_over_a_cached_prefix_matches_the_reference_kernel(vec):
    T, H, KVH, D = (int(v) for v in vec["prefill_dims"])
    scale = float(vec["prefill_scale"][0])
    info = vec["prefill_seqinfo"].reshape(-1, 4).astype(np.int64)
    for q_start, q_len, s_start, kv_len in info:
        own = vec["prefill_slots"][s_start:s_start + kv_len].astype(np.int64)
        prefix = kv_len - q_len
        # the new queries are the last q_len positions; positions before them have keys but need no query
        q_all = torch.zeros(kv_len, H, D, dtype=torch.float64)
        q_all[prefix:] = torch.from_numpy(vec["prefill_q"][q_start:q_start + q_len]).double()
        got = plain.causal_attention(q_all, torch.from_numpy(vec["prefill_k"][own]).double(),
                                     torch.from_numpy(vec["prefill_v"][own]).double(), scale)[prefix:]
        assert _rel(got.numpy(), vec["prefill_out"][q_start:q_start + q_len]) < 1e-5, (q_start, q_len)


def test_rms_norm_and_rotation_match_the_reference_kernel(vec):
    B, NH, Dm, HALF, K, R, n_keys = (int(v) for v in vec["qsa_dims"])
    eps = float(vec["qsa_eps"][0])
    keys = torch.from_numpy(vec["qsa_pool"][vec["qsa_slots"][:n_keys].astype(np.int64)]).double()      # key j sits at position j
    normed = plain.rms_norm(keys, torch.from_numpy(vec["qsa_knorm"]).double(), eps)
    rotated = plain.apply_rope(normed[:, None, :], torch.from_numpy(vec["qsa_cos"]).double(),
                               torch.from_numpy(vec["qsa_sin"]).double())[:, 0, :]
    # sequence i asked with +e_i, sequence Dm + i with -e_i: score = relu(+-rotated[j, i]) / sqrt(Dm)
    scores = vec["qsa_scores"].astype(np.float64)
    seen = (scores[:Dm] - scores[Dm:]).T * math.sqrt(Dm)                   # [key, dim]
    assert _rel(rotated.numpy(), seen) < 1e-5
    assert (scores >= 0).all() and ((scores[:Dm] == 0) | (scores[Dm:] == 0)).all()
    # the rotation really turned something, and left the dimensions beyond 2 * HALF alone
    assert np.abs(seen[1:, :2 * HALF] - normed.numpy()[1:, :2 * HALF]).max() > 0.1
    assert _rel(normed.numpy()[:, 2 * HALF:], seen[:, 2 * HALF:]) < 1e-5
    # the cos/sin tables the vectors were made with are the ones the plain implementation builds
    c, s = plain.rope_tables(torch.arange(n_keys), 2 * HALF, 10000.0)
    assert np.allclose(c.numpy(), vec["qsa_cos"], atol=1e-7) and np.allclose(s.numpy(), vec["qsa_sin"], atol=1e-7)


def test_sampler_uniforms_match_the_reference_kernel(vec):
    from carbon_engine_b200.sampling.sampler import mix64
    mask = (1 << 64) - 1
    for si, seed in enumerate(vec["uniform_seeds"].tolist()):
        for ii, i in enumerate(vec["uniform_idx"].tolist()):
            h = mix64(seed ^ mix64((i + 0x632BE59BD9B4E019) & mask))
            u = np.float32(np.float32(h >> 40) + np.float32(0.5)) * np.float32(1.0 / 16777216.0)
            assert u == vec["uniform_out"][si, ii], (seed, i)
    assert ((vec["uniform_out"] > 0) & (vec["uniform_out"] < 1)).all()


@pytest.mark.skipif(not os.environ.get("CARBON_REFERENCE_ROOT") or shutil.which("g++") is None,
                    reason="CARBON_REFERENCE_ROOT is not set (or there is no g++): the committed vectors are used as they are")
def test_committed_vectors_are_what_the_reference_sources_compute(vec, tmp_path):
    sys.path.insert(0, GOLDEN)
    import make_reference_vectors as maker
    fresh = str(tmp_path / "fresh.npz")
    maker.make(os.environ["CARBON_REFERENCE_ROOT"], fresh)
    again = np.load(fresh)
    assert sorted(again.files) == sorted(vec)
    for name in again.files:
        assert np.array_equal(again[name], vec[name]), name
