"""Host-side planning exported by the library: attention work items and replica sharding.
Integer work, so the checks are exact."""
import numpy as np

from oracle import generators as G


def test_attention_plan_covers_every_query_tile_once(lib):
    from tei_b200 import ops
    lens = [int(x) for x in G.lengths_cfg2()]
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    for causal in (False, True):
        work = ops.attention_plan(cu, causal)
        assert work.shape[0] == sum((n + 127) // 128 for n in lens)
        seen = set()
        for start, length, q0, _ in work.tolist():
            s = int(np.searchsorted(cu, start, side="right") - 1)
            assert cu[s] == start and lens[s] == length and q0 % 128 == 0 and q0 < length
            assert (s, q0) not in seen
            seen.add((s, q0))
        # most expensive first
        def cost(w):
            kv_end = min(w[1], w[2] + 128) if causal else w[1]
            return (kv_end + 127) // 128
        costs = [cost(w) for w in work.tolist()]
        assert costs == sorted(costs, reverse=True)


def test_attention_plan_edge_cases(lib):
    from tei_b200 import ops
    assert ops.attention_plan([0, 1], False).tolist() == [[0, 1, 0, 0]]
    assert ops.attention_plan([0, 128], False).tolist() == [[0, 128, 0, 0]]
    w = ops.attention_plan([0, 129], True).tolist()
    assert sorted(w) == [[0, 129, 0, 0], [0, 129, 128, 0]]


def test_attention_plan_with_a_sliding_window(lib):
    # flash_attn.rs:23-36: key j counts for query i when i - left <= j <= i + right.  The plan
    # stores the 64-aligned first key of each tile and orders tiles by their 64-key steps.
    from tei_b200 import ops
    lens = [1000, 5, 129, 300]
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    for causal, left, right in ((True, 100, -1), (False, 64, 64), (True, 0, -1), (False, -1, 10), (True, 5000, -1)):
        work = ops.attention_plan(cu, causal, left, right).tolist()
        assert len(work) == sum((n + 127) // 128 for n in lens)
        r = 0 if causal else right
        costs = []
        for start, length, q0, first in work:
            want_first = (max(0, q0 - left) // 64) * 64 if left >= 0 else 0
            assert first == want_first
            # no visible key of any row of the tile lies before `first`
            if left >= 0:
                assert first <= max(0, q0 - left)
            kv_end = min(length, q0 + 128 + r) if r >= 0 else length
            costs.append((kv_end - first + 63) // 64)
        assert costs == sorted(costs, reverse=True)
    # without a window the two entry points agree
    assert ops.attention_plan(cu, True, -1, -1).tolist() == ops.attention_plan(cu, True).tolist()


def test_plan_shards_balances_and_is_deterministic(lib):
    import tei_b200
    lens = G.lengths_cfg5()
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.uint32)
    a, b = 880.8e6 / 28, 2.0 * 2048  # per-layer linear and causal-attention cost
    for n in (1, 2, 4, 8):
        shard = tei_b200.plan_shards(cu, n, a, b)
        assert shard.min() >= 0 and shard.max() < n
        cost = a * lens + b * lens.astype(np.float64) ** 2
        loads = np.array([cost[shard == d].sum() for d in range(n)])
        # longest-first greedy: the spread is bounded by the largest single item
        assert loads.max() - loads.min() <= cost.max() + 1e-6
        assert (tei_b200.plan_shards(cu, n, a, b) == shard).all()
    one = tei_b200.plan_shards(cu, 1, a, b)
    assert (one == 0).all()


def test_gemm_tiling_follows_the_waves(lib):
    """Host arithmetic of the GEMM launch: CTA pairs wherever they fill the GPU, narrow
    single-CTA tiles only where the wide ones would leave most SMs without a tile (a wave of
    narrow tiles is hardly shorter than a wave of pairs: the main loop waits for its loads)."""
    t = lib.tei_b200_gemm_tiling
    sms = 148
    # the benchmark batches and their shards: pairs on every shape
    for m in (68576, 34288, 16384, 8572, 4096):
        for n in (2304, 768, 3072):
            assert t(m, n, sms, 1) == 0, (m, n)
    # one 512-token sequence: 2 x 3 pair tiles would use 12 of 148 SMs
    assert t(512, 768, sms, 1) == 64
    assert t(512, 2304, sms, 1) == 64
    assert t(512, 3072, sms, 1) == 128      # 192 tiles of 64 columns would need a second wave
    # 2,048 tokens: the pairs already fill one wave on the wide layers, not on the 768-column ones
    assert t(2048, 2304, sms, 1) == 0 and t(2048, 3072, sms, 1) == 0
    assert t(2048, 768, sms, 1) == 128
    # gated / rotary epilogues and device-side row counts have the 256-column tiles only
    assert t(512, 768, sms, 0) == 0
    assert t(100, 768, sms, 0) == 256       # at most 128 rows: no pair
    assert t(1, 768, sms, 1) == 64
    assert t(0, 768, sms, 1) == -1 and t(5, 0, sms, 1) == -1 and t(5, 5, 0, 1) == -1
