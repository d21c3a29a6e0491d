"""The routing-trace file format (no GPU): a trace written on a B200 by fomoe_b200_routing_trace_open is kept as a
fixture; the reference's reader (tools/read_trace.py) parsed it into routing_trace_expect.json.  This test checks that
the committed parser agrees with that parse field for field, that the reference's reader itself (when its tree is
present) still produces it, and the format's invariants: 32-byte header, 144-byte records at top-10
(the reference's routing_trace_record_t padded to 8 bytes)."""
import importlib.util
import json
import os

import numpy as np
import pytest

import helpers as H

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
BIN = os.path.join(GOLD, "routing_trace.bin")
REF_READER = os.path.join(os.environ.get("FOMOE_REF", "/root/reference"), "tools", "read_trace.py")


def _expect():
    with open(os.path.join(GOLD, "routing_trace_expect.json")) as f:
        return json.load(f)


def _same(mine, theirs):
    assert (mine["n_layers"], mine["n_experts"], mine["top_k"]) == (theirs["n_layers"], theirs["n_experts"], theirs["top_k"])
    assert len(mine["records"]) == len(theirs["records"])
    for a, b in zip(mine["records"], theirs["records"]):
        n = b["n_used"]
        assert (a["token"], a["layer"], a["n_used"], a["n_subs"]) == (b["token"], b["layer"], b["n_used"], b["n_subs"])
        for key in ("orig_ids", "final_ids", "source"):
            assert a[key][:n] == b[key]
        for key in ("orig_scores", "final_scores"):   # floats survive the JSON round trip exactly (repr of a double)
            assert np.array_equal(np.asarray(a[key][:n], dtype=np.float32), np.asarray(b[key], dtype=np.float32))


def test_fixture_layout():
    size = os.path.getsize(BIN)
    tr = H.parse_trace(BIN)
    assert tr["rec_size"] == 144 and tr["top_k"] == 10
    assert size == 32 + 144 * len(tr["records"]) and len(tr["records"]) == 15
    assert [(r["token"], r["layer"]) for r in tr["records"]] == [(t, l) for t in range(5) for l in range(3)]
    for r in tr["records"]:
        assert r["n_used"] == 10
        assert r["n_subs"] == sum(a != b for a, b in zip(r["orig_ids"], r["final_ids"]))
        assert all(0 <= e < tr["n_experts"] for e in r["orig_ids"] + r["final_ids"])
        assert all(s in (0, 2, 3, 4) for s in r["source"])
        assert all((s == 3) == (a != b) for s, a, b in zip(r["source"], r["orig_ids"], r["final_ids"]))
        assert abs(sum(r["orig_scores"]) - 1.0) < 1e-5
        assert all(x >= y for x, y in zip(r["orig_scores"], r["orig_scores"][1:]))   # ordered top-k
    assert sum(r["n_subs"] for r in tr["records"]) > 0


def test_committed_parser_agrees_with_reference_reader_output():
    _same(H.parse_trace(BIN), _expect())


@pytest.mark.skipif(not os.path.exists(REF_READER), reason="reference tree not present")
def test_reference_reader_parses_the_fixture():
    spec = importlib.util.spec_from_file_location("read_trace", REF_READER)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    live = mod.read_trace(BIN)
    assert live["n_tokens"] == 5
    _same(H.parse_trace(BIN), live)
    want = _expect()
    assert [r["final_ids"] for r in live["records"]] == [r["final_ids"] for r in want["records"]]
