"""Generates the golden fixtures in this directory by running the REFERENCE's own
compiled host code (``oracle/_ref``, see ``oracle/build_ref.py``) and the
``torch.nn.EmbeddingBag`` + ``torch.optim`` golden that the reference's operator
test uses (cust_op/test/split_embedding_codegen_lookup_adagrad_function_test/
torch/test_split_embedding_codegen_lookup_function.py:149-170) on seeded inputs.

Run from the repository root, in a container that has the reference tree:

    python oracle/build_ref.py && python tests/golden/make_golden.py

The fixtures are committed; the reference tree is not needed to run the tests.
"""
from __future__ import annotations

import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import ref  # noqa: E402
from tests.golden.driver import cache_driver_steps, run_cache_driver, zipf_ids  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))


# --------------------------------------------------------------------------- IdsMapper (A1, A2)
def golden_ids_mapper():
    t = ref.load_hybrid()
    rng = np.random.default_rng(101)
    T, steps = 3, 3
    out = {}
    mappers = [t.classes.hybrid.IdsMapper(4096, True) for _ in range(T)]
    for s in range(steps):
        lens = rng.integers(0, 400, size=T)
        lens[1] = 0 if s == 1 else lens[1]  # an empty table segment
        offset = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
        # raw keys: 63-bit values drawn from a small pool so steps share keys
        pool = rng.integers(0, 2**62, size=600, dtype=np.int64)
        ids = pool[rng.integers(0, 600, size=int(offset[-1]))]
        n = ids.size
        ids_t = torch.from_numpy(ids.copy())
        hi = torch.empty(n, dtype=torch.int64)
        uq = torch.empty(n, dtype=torch.int64)
        uid = torch.empty(n, dtype=torch.int64)
        inv = torch.empty(n, dtype=torch.int64)
        uoff = torch.zeros(T + 1, dtype=torch.int64)
        for tb in range(T):
            mappers[tb].ids2indices_unique_out(ids_t, hi, torch.from_numpy(offset), uq, uid, inv, uoff, tb)
        U = int(uoff[-1])
        out[f"s{s}_ids"] = ids
        out[f"s{s}_offset"] = offset
        out[f"s{s}_hash_indices"] = hi.numpy().copy()
        out[f"s{s}_unique"] = uq.numpy()[:U].copy()
        out[f"s{s}_unique_ids"] = uid.numpy()[:U].copy()
        out[f"s{s}_unique_inverse"] = inv.numpy().copy()
        out[f"s{s}_unique_offset"] = uoff.numpy().copy()
    # ids2indices_unique: slots + SORTED unique (UniqueParallel)
    m = t.classes.hybrid.IdsMapper(100000, True)
    for s in range(2):
        ids = zipf_ids(rng, 5000, 20000, 1.05) * 7919 + 13
        hi, uq, inv = m.ids2indices_unique(torch.from_numpy(ids))
        out[f"u{s}_ids"] = ids
        out[f"u{s}_hash_indices"] = hi.numpy().copy()
        out[f"u{s}_unique"] = uq.numpy().copy()
        out[f"u{s}_inverse"] = inv.numpy().copy()
    np.savez_compressed(os.path.join(OUT, "ids_mapper.npz"), **out)


# --------------------------------------------------------------------------- bucketize (A3)
def golden_bucketize():
    t = ref.load_hybrid()
    rng = np.random.default_rng(202)
    out = {}
    case = 0
    for W in (2, 4, 8):
        for do_unique, ret_count in ((False, False), (True, False), (True, True)):
            F, B = 3, 16
            lengths = rng.integers(0, 6, size=F * B).astype(np.int64)
            lengths[0] = max(lengths[0], 1)
            n = int(lengths.sum())
            indices = zipf_ids(rng, n, 500, 1.1)
            res = t.ops.hybrid.block_bucketize_sparse_features_cpu(
                torch.from_numpy(lengths), torch.from_numpy(indices), False, True,
                torch.ones(F, dtype=torch.int64), W, None, None, None, 0, None, False, False, do_unique, ret_count)
            out[f"c{case}_meta"] = np.array([W, F, B, int(do_unique), int(ret_count)], np.int64)
            out[f"c{case}_lengths"] = lengths
            out[f"c{case}_indices"] = indices
            out[f"c{case}_new_lengths"] = res[0].numpy().copy()
            out[f"c{case}_new_indices"] = res[1].numpy().copy()
            out[f"c{case}_unbucketize_permute"] = res[4].numpy().copy()
            out[f"c{case}_ids_counts"] = res[6].numpy().copy()
            case += 1
    out["n_cases"] = np.array([case], np.int64)
    np.savez_compressed(os.path.join(OUT, "bucketize.npz"), **out)


# --------------------------------------------------------------------------- cache slots / admit / evict (A4, A5)
def golden_cache():
    out = {}
    # case 0: roomy cache, admit >= 2, evict idle > 5 steps every 4 steps
    # case 1: tight cache (replacement sweep + reuse of evicted positions)
    # case 2: tight cache, no admit/evict (pure clock sweep)
    cases = [
        dict(cache=4096, admit=2, evict_thr=5, interval=4, steps=24, k=96, new=0.3, seed=9),
        dict(cache=160, admit=2, evict_thr=3, interval=3, steps=30, k=64, new=0.3, seed=10),
        dict(cache=200, admit=-1, evict_thr=0, interval=0, steps=30, k=64, new=0.4, seed=11),
    ]
    for ci, c in enumerate(cases):
        keys = cache_driver_steps(c["seed"], c["steps"], c["k"], c["new"])
        admit_on = c["admit"] != -1
        swap = ref.SwapManager(c["cache"], 1 if admit_on else 0)
        filt = ref.FeatureFilter(c["admit"], c["evict_thr"], c["interval"]) if (admit_on or c["evict_thr"]) else None
        rec = run_cache_driver(swap, filt, keys, c["interval"])
        out[f"c{ci}_meta"] = np.array([c["cache"], c["admit"], c["evict_thr"], c["interval"], c["steps"]], np.int64)
        for s, r in enumerate(rec):
            out[f"c{ci}_s{s}_keys"] = keys[s]
            for k, v in r.items():
                out[f"c{ci}_s{s}_{k}"] = v
    out["n_cases"] = np.array([len(cases)], np.int64)
    np.savez_compressed(os.path.join(OUT, "cache.npz"), **out)


# --------------------------------------------------------------------------- TBE forward / backward / optimizers (A6, A7)
def golden_tbe():
    """4 epochs of nn.EmbeddingBag(sparse=True) + torch.optim with loss = sum(out^2)/2,
    as the reference operator test does; records inputs, per-epoch outputs and final state."""
    out = {}
    torch.manual_seed(303)
    rng = np.random.default_rng(303)
    specs = [(200, 8), (300, 16), (120, 8)]
    B, epochs = 12, 4
    case = 0
    for mode in ("sum", "mean"):
        for opt in ("adagrad", "adam", "sgd"):
            bags = [torch.nn.EmbeddingBag(r, d, mode=mode, sparse=True, include_last_offset=True) for r, d in specs]
            for bag in bags:
                torch.nn.init.uniform_(bag.weight, -0.05, 0.05)
            params = [b.weight for b in bags]
            if opt == "adagrad":
                o = torch.optim.Adagrad(params, lr=0.05, eps=1e-8, initial_accumulator_value=0.1)
            elif opt == "adam":
                o = torch.optim.SparseAdam(params, lr=0.01, betas=(0.9, 0.999), eps=1e-8)
            else:
                o = torch.optim.SGD(params, lr=0.05)
            out[f"c{case}_w0"] = np.concatenate([b.weight.detach().numpy().reshape(-1) for b in bags])
            for e in range(epochs):
                idx_all, off_all, outs = [], [0], []
                for (r, d), bag in zip(specs, bags):
                    lens = rng.integers(0, 5, size=B)
                    idx = zipf_ids(rng, int(lens.sum()), r, 1.05)
                    offs = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
                    outs.append(bag(torch.from_numpy(idx), torch.from_numpy(offs)))
                    idx_all.append(idx)
                    off_all.extend((offs[1:] + off_all[-1]).tolist())  # feature-major [T*B+1]
                y = torch.cat(outs, dim=1)
                loss = (y * y).sum() / 2
                o.zero_grad()
                loss.backward()
                o.step()
                out[f"c{case}_e{e}_indices"] = np.concatenate(idx_all).astype(np.int64)
                out[f"c{case}_e{e}_offsets"] = np.array(off_all, np.int64)
                out[f"c{case}_e{e}_out"] = y.detach().numpy().copy()
            out[f"c{case}_w_final"] = np.concatenate([b.weight.detach().numpy().reshape(-1) for b in bags])
            out[f"c{case}_meta"] = np.array([0 if mode == "sum" else 1, {"adagrad": 1, "adam": 2, "sgd": 3}[opt], B,
                                             epochs], np.int64)
            case += 1
    out["specs"] = np.array(specs, np.int64)
    out["n_cases"] = np.array([case], np.int64)
    np.savez_compressed(os.path.join(OUT, "tbe_torch.npz"), **out)


if __name__ == "__main__":
    assert ref.available(), "build oracle/_ref first: python oracle/build_ref.py"
    golden_ids_mapper()
    golden_bucketize()
    golden_cache()
    golden_tbe()
    for f in sorted(os.listdir(OUT)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(OUT, f)))
