#!/usr/bin/env python3
"""Makes tests/golden/reference_vectors.npz: inputs, and what pedrosoares/carbon-engine's own kernel sources
compute for them when built for the CPU with reference_kernels_host.cpp.

    CARBON_REFERENCE_ROOT=<checkout of the reference> python tests/golden/make_reference_vectors.py [OUT.npz]

Four computations are recorded (tests/test_reference_anchor.py compares the plain implementation with
each of them):

* ``decode``:  src/kernels/attention.cu ``paged_decode_f32``: one query per sequence over a slot table;
* ``prefill``: src/kernels/attention.cu ``flash_prefill_f32``: new queries over a cached prefix and themselves;
* ``uniform``: src/kernels/sampling.cu ``carbon_uniform``: the sampler's counter-based random numbers;
* ``qsa``:     src/kernels/qsa.cu ``qsa_select_f32``, driven with one-hot queries so that its scratch scores
  spell out RMSNorm (with a weight) followed by the rotate-half rotation of a few keys.

The inputs are seeded, so a second run gives the same file.
"""
import os
import struct
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def build_driver(reference_root: str, out_dir: str) -> str:
    exe = os.path.join(out_dir, "ref_host")
    cmd = ["g++", "-std=c++20", "-O2", "-pthread", "-I", os.path.join(reference_root, "src", "kernels"),
           os.path.join(HERE, "reference_kernels_host.cpp"), "-o", exe]
    subprocess.run(cmd, check=True)
    return exe


def write_records(path, records):
    with open(path, "wb") as fh:
        for r in records:
            a = np.ascontiguousarray(r)
            assert a.dtype.itemsize == 4, a.dtype
            fh.write(struct.pack("<i", a.size))
            fh.write(a.tobytes())


def read_records(path, dtypes):
    out = []
    with open(path, "rb") as fh:
        for dt in dtypes:
            (n,) = struct.unpack("<i", fh.read(4))
            out.append(np.frombuffer(fh.read(4 * n), dtype=dt).copy())
    return out


def run(exe, mode, records, out_dtypes, tmp):
    src, dst = os.path.join(tmp, mode + ".in"), os.path.join(tmp, mode + ".out")
    write_records(src, records)
    subprocess.run([exe, mode, src, dst], check=True, timeout=600)
    return read_records(dst, out_dtypes)


def i32(v):
    return np.asarray([v], dtype=np.int32)


def f32(v):
    return np.asarray([v], dtype=np.float32)


def make_inputs():
    rng = np.random.default_rng(20240607)
    d = {}
    # ---- decode: 3 sequences of 1, 17 and 70 cached positions, 4 query heads on 2 KV heads of 32
    H, KVH, D, S = 4, 2, 32, 100
    lens = [1, 17, 70]
    perm = rng.permutation(S).astype(np.uint32)
    d["decode_dims"] = np.asarray([len(lens), H, KVH, D], dtype=np.int32)
    d["decode_scale"] = f32(1.0 / np.sqrt(D))
    d["decode_q"] = (rng.standard_normal((len(lens), H, D)) * 1.5).astype(np.float32)
    d["decode_k"] = (rng.standard_normal((S, KVH, D)) * 1.5).astype(np.float32)
    d["decode_v"] = rng.standard_normal((S, KVH, D)).astype(np.float32)
    d["decode_slots"] = perm[:sum(lens)]
    d["decode_starts"] = np.concatenate([[0], np.cumsum(lens)]).astype(np.uint32)
    # ---- prefill: a prefix of 5 with 37 new tokens, and 20 new tokens with no prefix
    S2 = 90
    perm2 = rng.permutation(S2).astype(np.uint32)
    seqs = [(5, 37), (0, 20)]          # (cached before, new)
    T = sum(n for _, n in seqs)
    d["prefill_dims"] = np.asarray([T, H, KVH, D], dtype=np.int32)
    d["prefill_scale"] = f32(1.0 / np.sqrt(D))
    d["prefill_q"] = (rng.standard_normal((T, H, D)) * 1.5).astype(np.float32)
    d["prefill_k"] = (rng.standard_normal((S2, KVH, D)) * 1.5).astype(np.float32)
    d["prefill_v"] = rng.standard_normal((S2, KVH, D)).astype(np.float32)
    info, tiles, q_start, s_start = [], [], 0, 0
    for b, (c, n) in enumerate(seqs):
        info += [q_start, n, s_start, c + n]          # q_start, q_len, slot_start, kv_len
        tiles += [[b, q0] for q0 in range(0, n, 64)]
        q_start += n
        s_start += c + n
    d["prefill_slots"] = perm2[:s_start]
    d["prefill_seqinfo"] = np.asarray(info, dtype=np.uint32)
    d["prefill_tiles"] = np.asarray(tiles, dtype=np.uint32).reshape(-1)
    # ---- uniform: 4 seeds x 9 indices, as (low word, high word) pairs
    seeds = np.asarray([0, 1, 0x9E3779B97F4A7C15, 0xFFFFFFFFFFFFFFFF], dtype=np.uint64)
    idx = np.asarray([0, 1, 2, 255, 256, 151935, 1 << 31, (1 << 32) + 5, (1 << 63) + 12345], dtype=np.uint64)
    d["uniform_seeds"] = seeds
    d["uniform_idx"] = idx
    # ---- qsa: 5 keys of 32 dims at positions 0..4, rotation over the first 16 dims; sequence b asks with
    # the query +e_b (b < 32) or -e_(b-32), so relu(q . key) reads one coordinate of the rotated key
    Dm, HALF, K, R, n_keys = 32, 8, 1, 1, 5
    B = 2 * Dm
    q = np.zeros((B, 1, Dm), dtype=np.float32)
    for i in range(Dm):
        q[i, 0, i] = 1.0
        q[Dm + i, 0, i] = -1.0
    theta = 10000.0
    inv_freq = theta ** (-2.0 * np.arange(HALF) / (2 * HALF))
    ang = np.arange(n_keys)[:, None] * inv_freq[None, :]
    d["qsa_dims"] = np.asarray([B, 1, Dm, HALF, K, R, n_keys], dtype=np.int32)
    d["qsa_eps"] = f32(1e-5)
    d["qsa_q"] = q
    d["qsa_pool"] = (rng.standard_normal((8, Dm)) * 2.0).astype(np.float32)
    d["qsa_knorm"] = (1.0 + 0.2 * rng.standard_normal(Dm)).astype(np.float32)
    d["qsa_cos"] = np.cos(ang).astype(np.float32)
    d["qsa_sin"] = np.sin(ang).astype(np.float32)
    key_slots = np.asarray([6, 2, 7, 0, 3], dtype=np.uint32)
    d["qsa_slots"] = np.tile(key_slots, B)
    d["qsa_starts"] = (np.arange(B + 1) * n_keys).astype(np.uint32)
    return d


def words(a64):
    """uint64 values as (low, high) uint32 pairs."""
    a64 = np.asarray(a64, dtype=np.uint64)
    return np.stack([a64 & np.uint64(0xFFFFFFFF), a64 >> np.uint64(32)], axis=1).astype(np.uint32).reshape(-1)


def compute(exe, d, tmp):
    out = {}
    dims = d["decode_dims"]
    (o,) = run(exe, "decode", [i32(dims[0]), i32(dims[1]), i32(dims[2]), i32(dims[3]), d["decode_scale"], d["decode_q"],
                               d["decode_k"], d["decode_v"], d["decode_slots"], d["decode_starts"]], [np.float32], tmp)
    out["decode_out"] = o.reshape(dims[0], dims[1], dims[3])
    dims = d["prefill_dims"]
    (o,) = run(exe, "prefill", [i32(dims[0]), i32(dims[1]), i32(dims[2]), i32(dims[3]), d["prefill_scale"], d["prefill_q"],
                                d["prefill_k"], d["prefill_v"], d["prefill_slots"], d["prefill_seqinfo"], d["prefill_tiles"]],
               [np.float32], tmp)
    out["prefill_out"] = o.reshape(dims[0], dims[1], dims[3])
    (u,) = run(exe, "uniform", [words(d["uniform_seeds"]), words(d["uniform_idx"])], [np.float32], tmp)
    out["uniform_out"] = u.reshape(len(d["uniform_seeds"]), len(d["uniform_idx"]))
    dims = d["qsa_dims"]
    scores, _, _ = run(exe, "qsa", [i32(v) for v in dims] + [d["qsa_eps"], d["qsa_q"], d["qsa_pool"], d["qsa_knorm"], d["qsa_cos"],
                                                             d["qsa_sin"], d["qsa_slots"], d["qsa_starts"]],
                       [np.float32, np.uint32, np.uint32], tmp)
    out["qsa_scores"] = scores.reshape(dims[0], dims[6])
    return out


def make(reference_root: str, out_path: str) -> None:
    with tempfile.TemporaryDirectory() as tmp:
        exe = build_driver(reference_root, tmp)
        d = make_inputs()
        d.update(compute(exe, d, tmp))
    np.savez_compressed(out_path, **d)


if __name__ == "__main__":
    root = os.environ.get("CARBON_REFERENCE_ROOT")
    if not root:
        sys.exit("set CARBON_REFERENCE_ROOT to a checkout of pedrosoares/carbon-engine")
    make(root, sys.argv[1] if len(sys.argv) > 1 else os.path.join(HERE, "reference_vectors.npz"))
