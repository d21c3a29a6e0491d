"""Writes routing_trace_expect.json: what the reference's own reader (tools/read_trace.py, imported from the reference
tree given as argv[1]) makes of routing_trace.bin.  routing_trace.bin itself was written on a B200 by
fomoe_b200_routing_trace_open / decode_token / tokens_run in tests/test_gpu_moe.py::test_routing_trace_and_expert_histogram
(run with FOMOE_KEEP_TRACE=<path> to keep a copy): 3 layers, 128 experts, top-10, CAR 0.35 with dampening, 5 tokens."""
import importlib.util
import json
import os
import sys

here = os.path.dirname(os.path.abspath(__file__))
spec = importlib.util.spec_from_file_location("read_trace", os.path.join(sys.argv[1], "tools", "read_trace.py"))
mod = importlib.util.module_from_spec(spec)
spec.loader.exec_module(mod)
tr = mod.read_trace(os.path.join(here, "routing_trace.bin"))
tr.pop("path")
with open(os.path.join(here, "routing_trace_expect.json"), "w") as f:
    json.dump(tr, f)
print(len(tr["records"]), "records,", tr["n_tokens"], "tokens")
