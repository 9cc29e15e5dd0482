"""Seeded operation sequences shared by the golden-vector generator, the CPU
oracle tests and the GPU parity tests.

A scenario is a table shape plus a list of steps; `run_scenario` plays it on
anything that offers the reference's method names with numpy arrays (the CPU
oracle, the CUDA product, the compiled reference) and returns one dict of
arrays per step, normalised so that legitimately order-dependent details
(slot positions, the order of exported or evicted tuples) do not show.

Every batch holds unique keys.  Where a batch can evict, its scores are
distinct and larger than every score already stored, so the surviving set is
independent of the order in which a parallel implementation applies the batch.
"""
from __future__ import annotations

import numpy as np

from tests.hkv_testlib import sorted_by_key, unique_keys, values_for

LRU, LFU, EPOCH_LRU, EPOCH_LFU, CUSTOMIZED = range(5)
TIME_SCORED = (LRU, EPOCH_LRU)


def _scores(start: int, n: int) -> np.ndarray:
    return np.arange(start, start + n, dtype=np.uint64)


def build_scenarios() -> dict:
    sc = {}
    cap, dim = 8192, 4
    keys = unique_keys(40000, seed=101)

    # -- Customized: fill without eviction, look up, assign family, erase -------
    a, b, fresh = keys[:2048], keys[2048:4096], keys[4096:5120]
    sc["customized_basic"] = dict(capacity=cap, dim=dim, strategy=CUSTOMIZED, steps=[
        ("insert_or_assign", a, _scores(1, a.size)),
        ("insert_or_assign", b, _scores(10001, b.size)),
        ("size",),
        ("find", np.concatenate([a[:512], fresh[:512], b[:512]])),
        ("contains", np.concatenate([fresh[:300], a[:300]])),
        ("insert_or_assign", a[:1024], _scores(20001, 1024)),        # pure assign
        ("assign", np.concatenate([b[:256], fresh[:256]]), _scores(30001, 512)),
        ("assign_scores", np.concatenate([a[1024:1280], fresh[256:512]]), _scores(40001, 512)),
        ("find", np.concatenate([a, b])),
        ("export",),
        ("export_if", 1, 0, 20001),   # score < 20001
        ("export_if", 2, 0, 20001),   # score >= 20001
        ("export_if", 3, 0x5, 0xF),   # (key & 0xF) == 5
        ("erase", np.concatenate([a[:700], fresh[:100]])),
        ("size",),
        ("find", a[:1400]),
        ("insert_or_assign", fresh[:600], _scores(50001, 600)),       # reuses tombstones or empties
        ("size",),
        ("export",),
    ])

    # -- Customized: overfill, min-score eviction, refusal ---------------------------
    steps = []
    base = 1
    for r in range(5):
        k = keys[6000 + r * 4096: 6000 + (r + 1) * 4096]
        steps.append(("insert_or_assign", k, _scores(base, k.size)))
        base += 10000
        steps.append(("size",))
    low = keys[30000:31024]
    steps.append(("insert_or_assign", low, _scores(1, low.size)))      # all refused: scores too low
    steps.append(("size",))
    steps.append(("find", np.concatenate([low[:256], keys[6000 + 4 * 4096: 6000 + 4 * 4096 + 256]])))
    steps.append(("export",))
    sc["customized_evict"] = dict(capacity=cap, dim=dim, strategy=CUSTOMIZED, steps=steps)

    # -- insert_and_evict: evicted and refused tuples come back ------------------------
    steps = []
    base = 1000
    for r in range(4):
        k = keys[6000 + r * 4096: 6000 + (r + 1) * 4096]
        steps.append(("insert_and_evict", k, _scores(base, k.size)))
        base += 10000
    steps.append(("insert_and_evict", keys[31024:32048], _scores(1, 1024)))   # refused inputs
    steps.append(("size",))
    steps.append(("export",))
    sc["customized_insert_and_evict"] = dict(capacity=cap, dim=dim, strategy=CUSTOMIZED, steps=steps)

    # -- find_or_insert / accum_or_assign ------------------------------------------------
    c = keys[32048:34096]
    mix = np.concatenate([c[:1024], keys[34096:35120]])
    flags = np.zeros(mix.size, dtype=np.bool_)
    flags[::2] = True
    sc["customized_find_or_insert_accum"] = dict(capacity=cap, dim=dim, strategy=CUSTOMIZED, steps=[
        ("insert_or_assign", c, _scores(1, c.size)),
        ("find_or_insert", mix, _scores(5001, mix.size)),     # half hits (rows come back), half inserts
        ("export",),
        ("accum_or_assign", mix, flags, _scores(9001, mix.size)),
        ("accum_or_assign", keys[35120:35632], np.tile(np.array([True, False]), 256),
         _scores(12001, 512)),                                  # accum on misses is a no-op
        ("export",),
        ("size",),
    ])

    # -- Lfu: scores add up on a hit ----------------------------------------------------------
    d = keys[36000:38048]
    freq = (d % np.uint64(1000)) + np.uint64(1)
    sc["lfu"] = dict(capacity=cap, dim=dim, strategy=LFU, steps=[
        ("insert_or_assign", d, freq),
        ("insert_or_assign", d[:1024], freq[:1024]),
        ("assign", d[1024:1536], freq[1024:1536]),
        ("find", d),
        ("export",),
    ])

    # -- EpochLfu: epoch in the high half, saturating frequency in the low half ---------------
    e = keys[38048:39072]
    big = np.full(256, 0xFFFFFFF0, dtype=np.uint64)
    sc["epoch_lfu"] = dict(capacity=cap, dim=dim, strategy=EPOCH_LFU, steps=[
        ("set_epoch", 3),
        ("insert_or_assign", e, (e % np.uint64(100)) + np.uint64(1)),
        ("set_epoch", 4),
        ("insert_or_assign", e[:512], (e[:512] % np.uint64(7)) + np.uint64(1)),
        ("insert_or_assign", e[512:768], big),
        ("insert_or_assign", e[512:768], big),                        # saturates at 0xFFFFFFFF
        ("set_epoch", 6),
        ("assign", e[768:900], (e[768:900] % np.uint64(5)) + np.uint64(1)),
        ("find", e),
        ("export_if", 1, 0, 4 << 32),                                 # score < epoch 4
        ("export",),
    ])

    # -- Lru / EpochLru: timer scores, only hit/miss sets and rows are comparable -----------------
    f = keys[:3000]
    sc["lru"] = dict(capacity=cap, dim=dim, strategy=LRU, steps=[
        ("insert_or_assign", f[:2000], None),
        ("insert_or_assign", f[1500:3000], None),
        ("find", keys[1000:4000]),
        ("size",),
        ("export",),
    ])
    sc["epoch_lru"] = dict(capacity=cap, dim=dim, strategy=EPOCH_LRU, steps=[
        ("set_epoch", 9),
        ("insert_or_assign", f[:2000], None),
        ("find_or_insert", f[1500:3000], None),
        ("find", keys[1000:4000]),
        ("export",),
    ])

    # -- reserved_key_start_bit moves the reserved keys -----------------------------------------
    g = unique_keys(1500, seed=202, reserved_key_start_bit=17)
    odd = np.array([0xFFFFFFFFFFFFFFFF, 0xFFFFFFFFFFFFFFFE, 0xFFFFFFFFFFFFFFFD,
                    0xFFFFFFFFFFFFFFFC], dtype=np.uint64)      # ordinary keys when the bit is 17
    rsv = np.array([0xFFFFFFFFFFFFFFFE, 0xFFFFFFFFFFFDFFFE, 0xFFFFFFFFFFFBFFFE,
                    0xFFFFFFFFFFF9FFFE], dtype=np.uint64)       # the four reserved keys for bit 17
    gk = np.concatenate([g[:1000], odd[[0, 2, 3]], rsv[1:]])
    sc["reserved_bit_17"] = dict(capacity=cap, dim=dim, strategy=CUSTOMIZED,
                                 reserved_key_start_bit=17, steps=[
        ("insert_or_assign", gk, _scores(1, gk.size)),
        ("size",),
        ("find", np.concatenate([gk, g[1000:1200]])),
        ("export",),
    ])

    # -- a table that grows: auto-rehash on the insert path, reserve, set_max_capacity ------
    w = unique_keys(30000, seed=303)
    steps = [("capacity",)]
    at = 0
    for r, n in enumerate([300, 300, 500, 900]):       # 1024 -> 2048 -> 4096 along the way
        steps += [("insert_or_assign", w[at:at + n], _scores(1 + at, n)), ("capacity",)]
        at += n
    steps += [
        ("erase", w[100:600]),                          # tombstones do not survive a rehash
        ("size",),
        ("reserve", 8192), ("capacity",), ("size",),
        ("find", w[:2200]),
        ("export",),
        ("reserve", 1 << 20), ("capacity",),            # above max_capacity: ignored
        ("find_or_insert", w[at:at + 3000], _scores(1 + at, 3000)), ("capacity",),
    ]
    at += 3000
    for r in range(6):                                  # reaches 16384, then overfills it
        steps += [("insert_or_assign", w[at:at + 2500], _scores(1 + at, 2500)), ("capacity",)]
        at += 2500
    steps += [
        ("size",),
        ("find", w[:at]),
        ("set_max_capacity_rejected", 40000),           # not a power of two
        ("set_max_capacity", 8192), ("capacity",),      # below the capacity: ignored
        ("insert_or_assign", w[at:at + 1000], _scores(1 + at, 1000)), ("capacity",),
        ("set_max_capacity", 65536),                    # growth resumes
        ("insert_and_evict", w[at + 1000:at + 3000], _scores(1001 + at, 2000)), ("capacity",),
        ("accum_or_assign", w[at + 3000:at + 4000], np.zeros(1000, dtype=bool),
         _scores(3001 + at, 1000)),
        ("capacity",), ("size",),
        ("find", w[:at + 4000]),
        ("export",),
    ]
    sc["customized_growth"] = dict(capacity=1024, max_capacity=16384, max_load_factor=0.5,
                                   dim=dim, strategy=CUSTOMIZED, steps=steps)
    return sc


def table_kwargs(scenario: dict) -> dict:
    """Constructor keywords of OracleTable / ProductTable / RefTable beyond
    (capacity, dim, strategy)."""
    kw = {"reserved_key_start_bit": scenario.get("reserved_key_start_bit", 0)}
    for name in ("max_capacity", "max_load_factor"):
        if name in scenario:
            kw[name] = scenario[name]
    return kw


def run_scenario(table, scenario: dict) -> list:
    """Plays the steps on `table`; returns one dict of numpy arrays per step."""
    dim = scenario["dim"]
    timed = scenario["strategy"] in TIME_SCORED
    out = []
    for idx, step in enumerate(scenario["steps"]):
        op = step[0]
        res = {}
        if op == "set_epoch":
            table.set_global_epoch(step[1])
        elif op == "insert_or_assign":
            table.insert_or_assign(step[1], values_for(step[1], dim, seed=idx), step[2])
        elif op == "size":
            res["size"] = np.array([table.size()], dtype=np.uint64)
        elif op == "capacity":
            res["capacity"] = np.array([table.capacity()], dtype=np.uint64)
        elif op == "reserve":
            table.reserve(step[1])
        elif op == "set_max_capacity":
            table.set_max_capacity(step[1])
        elif op == "set_max_capacity_rejected":
            try:
                table.set_max_capacity(step[1])
                res["rejected"] = np.array([0], dtype=np.uint64)
            except ValueError:
                res["rejected"] = np.array([1], dtype=np.uint64)
        elif op == "find":
            v, f, s = table.find(step[1])
            res["founds"] = f
            res["values"] = v[f]
            if not timed:
                res["scores"] = s[f]
        elif op == "contains":
            res["founds"] = table.contains(step[1])
        elif op == "find_or_insert":
            vals = values_for(step[1], dim, seed=idx)
            res["values"] = table.find_or_insert(step[1], vals, step[2])
        elif op == "insert_and_evict":
            ek, ev, es = table.insert_and_evict(step[1], values_for(step[1], dim, seed=idx), step[2])
            ek, ev, es = sorted_by_key(ek, ev, es)
            res["evicted_keys"], res["evicted_values"] = ek, ev
            if not timed:
                res["evicted_scores"] = es
        elif op == "accum_or_assign":
            table.accum_or_assign(step[1], values_for(step[1], dim, seed=idx), step[2], step[3])
        elif op == "assign":
            table.assign(step[1], values_for(step[1], dim, seed=idx), step[2])
        elif op == "assign_scores":
            table.assign_scores(step[1], step[2])
        elif op == "erase":
            table.erase(step[1])
        elif op in ("export", "export_if"):
            if op == "export":
                k, v, s = table.export_batch()
            else:
                k, v, s = table.export_batch_if(step[1], step[2], step[3])
            k, v, s = sorted_by_key(k, v, s)
            res["keys"], res["values"] = k, v
            if not timed:
                res["scores"] = s
        else:
            raise ValueError(op)
        out.append(res)
    return out


def flatten(results: list) -> dict:
    """{ 'step03.keys': array, ... } for np.savez."""
    flat = {}
    for i, res in enumerate(results):
        for name, arr in res.items():
            flat[f"step{i:02d}.{name}"] = arr
    return flat


def compare(got: list, want: list, label: str) -> None:
    assert len(got) == len(want), label
    for i, (g, w) in enumerate(zip(got, want)):
        assert set(g) == set(w), f"{label} step {i}: {sorted(g)} vs {sorted(w)}"
        for name in w:
            a, b = np.asarray(g[name]), np.asarray(w[name])
            if a.dtype == np.float32:
                a, b = a.view(np.uint32), b.astype(np.float32).view(np.uint32)
            np.testing.assert_array_equal(a, b, err_msg=f"{label} step {i} {name}")
