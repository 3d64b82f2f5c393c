"""TEST INFRASTRUCTURE - CPU restatement of the reference's device gate.

Only tests/, `__graft_entry__.smoke()` and bench.py's cpu_baseline / reference legs may import
this package; the product path never does.

`compute_cap_matching` follows backends/candle/src/compute_cap.rs:27-40: whether a binary built
for `compile_cap` may run on a device of `runtime_cap` (both as major * 10 + minor).  The
reference refuses to start otherwise (backends/candle/src/lib.rs:240-248).  Pinned by the
reference's own assertions (compute_cap.rs:53-110), replayed in tests/test_capability.py.
"""


def compute_cap_matching(runtime_cap: int, compile_cap: int) -> bool:
    r, c = runtime_cap, compile_cap
    return ((r == 75 and c == 75)
            or (80 <= r <= 89 and c == 80)
            or (86 <= r <= 89 and 80 <= c <= 86)
            or (r == 89 and c == 89)
            or (r == 90 and c == 90)
            or (r == 100 and c == 100)
            or (120 <= r <= 121 and c == 120)
            or (r == 121 and c == 121))
