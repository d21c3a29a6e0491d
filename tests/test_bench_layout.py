"""Host logic of the benchmark: how ranks map onto tensor-parallel groups, and the workload record."""
import importlib.util
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
    m = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(m)
    return m


def test_rank_layout():
    b = _bench()
    assert b.tp_layout(1) == (1, 1, 0, 0)
    assert [b.tp_layout(2, r) for r in range(2)] == [(2, 1, 0, 0), (2, 1, 0, 1)]
    assert [b.tp_layout(4, r)[2:] for r in range(4)] == [(0, 0), (0, 1), (0, 2), (0, 3)]
    lay = [b.tp_layout(8, r) for r in range(8)]
    assert all(t == 4 and n == 2 for t, n, _, _ in lay)                  # two groups of four
    assert [g for _, _, g, _ in lay] == [0, 0, 0, 0, 1, 1, 1, 1]          # consecutive ranks form a group
    assert [r for _, _, _, r in lay] == [0, 1, 2, 3, 0, 1, 2, 3]


def test_workload_record_and_bytes():
    b = _bench()
    assert b.expert_bytes_per_token(12) == 1005649920                    # 6 x 89,751,552 + 6 x 77,856,768
    assert b.expert_bytes_per_token(60) == 5028249600
    c1, c8 = b.workload_config(1, 12, 256), b.workload_config(8, 60, 128)
    assert c1["parallelism"] == "tp1" and "first 12 of 60 layers" in c1["workload"]
    assert c8["parallelism"].startswith("2 independent batch-1 streams x tp4")
    assert set(c1) == set(c8)
