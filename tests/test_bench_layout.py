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
    assert all(t == 8 and n == 1 and g == 0 for t, n, g, _ in lay)       # one stream over all eight GPUs
    assert [r for _, _, _, r in lay] == list(range(8))
    rep = [b.tp_layout(8, r, 4) for r in range(8)]                        # --tp 4: two replicas, comparison only
    assert all(t == 4 and n == 2 for t, n, _, _ in rep)
    assert [g for _, _, g, _ in rep] == [0, 0, 0, 0, 1, 1, 1, 1]          # consecutive ranks form a group
    assert [r for _, _, _, r in rep] == [0, 1, 2, 3, 0, 1, 2, 3]


def test_workload_record_and_bytes():
    b = _bench()
    assert b.expert_bytes_per_token(12) == 1005649920                    # 6 x 89,751,552 + 6 x 77,856,768
    assert b.expert_bytes_per_token(60) == 5028249600
    c1, c8 = b.workload_config(1, 12, 256), b.workload_config(8, 60, 128)
    assert c1["parallelism"] == "tp1" and "first 12 of 60 layers" in c1["workload"]
    assert c8["parallelism"] == "tp8"
    assert b.workload_config(8, 60, 128, 4)["parallelism"].startswith("2 replicas x tp4")
    assert set(c1) == set(c8)


def test_reference_arm_runs_without_the_cuda_library():
    """`bench.py --impl reference` prints a line whose config equals the GPU arm's for the same arguments, takes its
    inputs from the host-only generator, and never maps libfomoe_b200.so."""
    import json
    import subprocess
    import sys
    code = ("import sys, runpy; sys.argv = ['bench.py', '--impl', 'reference', '--steps', '2', '--warmup', '0'];\n"
            "import bench; bench.cpu_baseline.__defaults__ = (None, 2, 0.05)\n"
            "bench.main()\n"
            "maps = open('/proc/self/maps').read()\n"
            "print('MAPPED_PRODUCT', 'libfomoe_b200.so' in maps, 'libfomoe_synth.so' in maps)\n")
    out = subprocess.run([sys.executable, "-c", code], cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = out.stdout.strip().splitlines()
    line = json.loads(next(l for l in lines if l.startswith("{")))
    assert line["impl"] == "reference" and line["cpu_baseline"]["kind"] in ("reference", "port")
    assert line["config"] == _bench().workload_config(1, 12, 2)
    assert "MAPPED_PRODUCT False True" in lines[-1]


def test_reference_arm_of_the_batched_configuration():
    """`bench.py --impl reference --config 4`: the reference's per-token CPU path on the batched configuration's layer,
    same metric, unit and workload string as the GPU arm's line, host-only inputs (the logits of the host generator
    equal the ones the library generates on the device)."""
    import json
    import subprocess
    import sys
    code = ("import sys; sys.argv = ['bench.py', '--impl', 'reference', '--config', '4', '--steps', '2', '--warmup', '0'];\n"
            "import bench; bench.cpu_baseline4.__defaults__ = (None, 2, 0.05)\n"
            "bench.main()\n"
            "maps = open('/proc/self/maps').read()\n"
            "print('MAPPED_PRODUCT', 'libfomoe_b200.so' in maps, 'libfomoe_synth.so' in maps)\n")
    out = subprocess.run([sys.executable, "-c", code], cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = out.stdout.strip().splitlines()
    line = json.loads(next(l for l in lines if l.startswith("{")))
    b = _bench()
    assert line["impl"] == "reference" and line["metric"] == b.C4_METRIC and line["unit"] == b.C4_UNIT
    assert line["config"] == {"workload": b.c4_workload(48)} and line["value"] > 0
    assert "MAPPED_PRODUCT False True" in lines[-1]
    import numpy as np
    import fomoe_b200
    from fomoe_b200 import synth
    assert (fomoe_b200.synth_logits(7, 2, 5, 16).reshape(-1) == synth.f32(7, 2, 8, 0.0, 1.0, 5 * 16)).all()


def test_host_generator_library_matches_the_main_library(fb=None):
    import numpy as np
    import fomoe_b200
    from fomoe_b200 import synth
    a = fomoe_b200.synth_expert_record(5, 1, 3, 14, 512, 256)
    assert (a == synth.expert_record(5, 1, 3, 14, 512, 256)).all()
    assert (fomoe_b200.synth_hidden(5, 2, 512) == synth.hidden(5, 2, 512)).all()
    assert (fomoe_b200.synth_router(5, 1, 8, 512) == synth.router(5, 1, 8, 512)).all()
    for x, y in zip(fomoe_b200.synth_glue(5, 1, 512), synth.glue(5, 1, 512)):
        assert (x == y).all()
    assert (fomoe_b200.synth_matrix(9, 0, 1, 2, 13, 256, 512) == synth.matrix(9, 0, 1, 2, 13, 256, 512)).all()
