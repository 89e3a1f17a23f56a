"""Seeded input streams and the per-step call order shared by the fixture generator
(make_golden.py) and the parity tests.  Pure numpy; imports nothing else from this repo."""
from __future__ import annotations

import numpy as np


def zipf_ids(rng, n, vocab, alpha):
    ranks = np.arange(1, vocab + 1, dtype=np.float64)
    p = ranks ** (-alpha)
    p /= p.sum()
    return rng.choice(vocab, size=n, p=p).astype(np.int64)



def cache_driver_steps(seed, steps, keys_per_step, new_rate, key_bits=62):
    """The seeded key stream of the dynamic-table config, scaled down: each step has
    ``new_rate`` fresh uniform keys and the rest resampled from keys issued so far."""
    rng = np.random.default_rng(seed)
    issued = rng.integers(0, 2**key_bits, size=keys_per_step, dtype=np.int64)
    out = []
    for s in range(steps):
        n_new = int(round(keys_per_step * new_rate)) if s > 0 else keys_per_step
        fresh = rng.integers(0, 2**key_bits, size=n_new, dtype=np.int64)
        old = issued[rng.integers(0, issued.size, size=keys_per_step - n_new)]
        keys = np.concatenate([fresh, old])
        rng.shuffle(keys)
        issued = np.concatenate([issued, fresh])
        out.append(keys)
    return out


def first_occurrence_unique(keys):
    _, first = np.unique(keys, return_index=True)
    return keys[np.sort(first)]


def run_cache_driver(swap, filt, steps_keys, evict_interval):
    """record_timestamp -> (evict) -> statistics -> first-occurrence unique ->
    count_filter -> compute_swap_info, per step; returns per-step outputs."""
    rec = []
    for s, keys in enumerate(steps_keys):
        ts = np.full(keys.size, s, np.int64)
        evicted = np.empty(0, np.int64)
        if filt is not None:
            filt.record_timestamp(keys, ts)
            if evict_interval and s > 0 and (s + 1) % evict_interval == 0:
                evicted = filt.evict_keys()
                swap.remove_keys(evicted)
                filt.clear_evict()
            filt.statistics_key_count(keys)
        uniq = first_occurrence_unique(keys)
        filtered = filt.count_filter(uniq) if filt is not None else uniq
        so_k, so_o, si_k, si_o, bo = swap.compute_swap_info(filtered)
        rec.append(dict(filtered=filtered, evicted=np.sort(evicted), swapout_keys=so_k, swapout_offs=so_o,
                        swapin_keys=si_k, swapin_offs=si_o, batch_offs=bo))
    return rec
